// Symmetric (peer-mapped) device memory for the fused multi-GPU kernels.
//
// Each rank allocates its buffer with cudaMalloc, exports a CUDA IPC handle, and opens the
// handles of its peers; the Python side (parallel/symm.py) moves the 64-byte handles through
// the process group.  Kernels then address peers' memory with ordinary loads and stores over
// NVLink.  No multicast object is ever created or bound here, so a rank that exits does not
// leave peers attached to a multicast group.  (The reference has no communication layer of its
// own; it calls torch.distributed collectives, apexw/zero.py:300-338.)
//
// Lifetime: an allocation is a reference-counted object.  Every tensor made over it (and so
// every view of such a tensor: model parameters and gradients that were re-pointed into the
// flat buffers) holds a reference through the deleter of its storage.  The memory is released
// when the last reference goes - the Python handle, or the last tensor storage, whichever
// lives longer - so dropping an optimizer never leaves parameters pointing at freed memory.
#include <torch/extension.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <atomic>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

namespace {

void ok(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, what, " failed: ", cudaGetErrorString(e)); }

std::atomic<int64_t> g_live_allocations{0};
std::atomic<int64_t> g_live_bytes{0};

class SymmAlloc {
  public:
    SymmAlloc(int64_t nbytes, int64_t device) : nbytes_(nbytes), device_(device) {
        TORCH_CHECK(nbytes > 0, "SymmAlloc: size must be positive");
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
        ok(cudaMalloc(&ptr_, static_cast<size_t>(nbytes)), "cudaMalloc");
        ok(cudaMemset(ptr_, 0, static_cast<size_t>(nbytes)), "cudaMemset");
        ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        ok(cudaIpcGetMemHandle(&handle_, ptr_), "cudaIpcGetMemHandle");
        g_live_allocations.fetch_add(1);
        g_live_bytes.fetch_add(nbytes_);
    }
    SymmAlloc(const SymmAlloc&) = delete;
    SymmAlloc& operator=(const SymmAlloc&) = delete;

    // Runs when the last holder (Python handle or tensor storage) lets go.  Peer mappings are closed before
    // the local memory is released.  No error is raised from here: at interpreter shutdown the context may
    // already be gone.
    ~SymmAlloc() {
        int prev = -1;
        const bool switched = cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(static_cast<int>(device_)) == cudaSuccess;
        if (switched) {
            cudaDeviceSynchronize();
            for (void* p : opened_) cudaIpcCloseMemHandle(p);
            cudaFree(ptr_);
            cudaSetDevice(prev);
        }
        cudaGetLastError();
        g_live_allocations.fetch_sub(1);
        g_live_bytes.fetch_sub(nbytes_);
    }

    int64_t ptr() const { return reinterpret_cast<int64_t>(ptr_); }
    int64_t nbytes() const { return nbytes_; }
    int64_t device() const { return device_; }
    pybind11::bytes handle() const { return pybind11::bytes(reinterpret_cast<const char*>(&handle_), sizeof(handle_)); }

    // Map a peer's allocation (its exported handle) into this process; the mapping lives as long as this object.
    int64_t open_peer(const std::string& handle) {
        TORCH_CHECK(handle.size() == sizeof(cudaIpcMemHandle_t), "open_peer: bad handle size");
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_));
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handle.data(), sizeof(h));
        void* p = nullptr;
        ok(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
        opened_.push_back(p);
        return reinterpret_cast<int64_t>(p);
    }

  private:
    void* ptr_ = nullptr;
    int64_t nbytes_;
    int64_t device_;
    cudaIpcMemHandle_t handle_;
    std::vector<void*> opened_;
};

// Tensor over [ptr, ptr + bytes of shape) that keeps `owner` alive through its storage.  `ptr` is either inside
// the owner's own memory or inside one of its peer mappings (both die with the owner).
at::Tensor symm_tensor(std::shared_ptr<SymmAlloc> owner, int64_t ptr, std::vector<int64_t> shape, at::ScalarType dtype) {
    TORCH_CHECK(owner != nullptr, "symm_tensor: no allocation");
    auto opts = at::TensorOptions().dtype(dtype).device(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(owner->device())));
    return at::from_blob(reinterpret_cast<void*>(ptr), shape, [owner](void*) mutable { owner.reset(); }, opts);
}

// Non-owning tensor over raw device memory; the caller keeps the memory alive (tests and tools).
at::Tensor tensor_from_ptr(int64_t ptr, std::vector<int64_t> shape, at::ScalarType dtype, int64_t device) {
    auto opts = at::TensorOptions().dtype(dtype).device(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device)));
    return at::from_blob(reinterpret_cast<void*>(ptr), shape, [](void*) {}, opts);
}

bool can_access_peer(int64_t device, int64_t peer) {
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, static_cast<int>(device), static_cast<int>(peer)) != cudaSuccess) return false;
    return can != 0;
}

}  // namespace

void register_symm(pybind11::module_& m) {
    pybind11::class_<SymmAlloc, std::shared_ptr<SymmAlloc>>(m, "SymmAlloc")
        .def(pybind11::init<int64_t, int64_t>(), pybind11::arg("nbytes"), pybind11::arg("device"))
        .def_property_readonly("ptr", &SymmAlloc::ptr)
        .def_property_readonly("nbytes", &SymmAlloc::nbytes)
        .def_property_readonly("handle", &SymmAlloc::handle)
        .def("open_peer", &SymmAlloc::open_peer);
    m.def("symm_tensor", &symm_tensor);
    m.def("symm_live_allocations", []() { return g_live_allocations.load(); });
    m.def("symm_live_bytes", []() { return g_live_bytes.load(); });
    m.def("tensor_from_ptr", &tensor_from_ptr);
    m.def("can_access_peer", &can_access_peer);
    m.attr("max_peers") = 8;
    m.attr("signal_words") = 18;
}

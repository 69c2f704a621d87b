// Host side of the tcgen05 Newton-Schulz path: tensor-map construction and the iteration driver.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <vector>
#include "api.h"

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        TORCH_CHECK(e == cudaSuccess && p != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
        fn = reinterpret_cast<EncodeFn>(p);
    }
    return fn;
}

// bf16 tensor [batch, rows, cols] (cols contiguous) -> map with box {64 cols, box_rows rows, 1}
CUtensorMap make_map(const at::Tensor& t, int box_rows) {
    TORCH_CHECK(t.dim() == 3 && t.is_contiguous() && t.scalar_type() == at::kBFloat16, "expected contiguous bf16 [batch, rows, cols]");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0 && (t.size(2) * 2) % 16 == 0, "tensor map needs 16-byte aligned rows");
    CUtensorMap m;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(t.size(2)), static_cast<cuuint64_t>(t.size(1)), static_cast<cuuint64_t>(t.size(0))};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(t.size(2)) * 2, static_cast<cuuint64_t>(t.size(1)) * t.size(2) * 2};
    const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, t.data_ptr(), dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", static_cast<int>(r));
    return m;
}

void gemm(const at::Tensor& A, const at::Tensor& B, const c10::optional<at::Tensor>& D, at::Tensor& C,
          c10::optional<at::Tensor> Ct, float alpha, float beta, at::Tensor& err, bool symmetric = false, int force_bn = 0) {
    const int batch = static_cast<int>(A.size(0)), M = static_cast<int>(A.size(1)), K = static_cast<int>(A.size(2));
    const int N = static_cast<int>(B.size(1));
    TORCH_CHECK(B.size(0) == batch && B.size(2) == K, "operand shapes disagree");
    TORCH_CHECK(C.size(0) == batch && C.size(1) == M && C.size(2) == N && C.is_contiguous(), "output shape");
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const int bn = force_bn ? force_bn : apexb_ns_pick_tile(M, N, K, batch, symmetric ? 1 : 0, sms);
    TORCH_CHECK(bn == 128 || bn == 256 || bn == 512, "tile selector must be 128, 256 or 512 (512: 256 x 256 tiles on CTA pairs)");
    const CUtensorMap ma = make_map(A, 128);
    const CUtensorMap mb = make_map(B, bn == 512 ? 128 : bn);     // a CTA of a pair loads its own 128 rows of B
    const void* d = (D.has_value() && D->defined()) ? D->data_ptr() : nullptr;
    void* ct = (Ct.has_value() && Ct->defined()) ? Ct->data_ptr() : nullptr;
    if (symmetric) {
        TORCH_CHECK(M == N, "a symmetric product is square");
        ct = C.data_ptr();
    }
    int rc = apexb_ns_gemm(&ma, &mb, d, C.data_ptr(), ct, static_cast<long long>(M) * N, static_cast<long long>(M) * N,
                           static_cast<long long>(M) * N, M, N, K, batch, alpha, beta, symmetric ? 1 : 0, bn, sms,
                           reinterpret_cast<unsigned*>(err.data_ptr<int>()), at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == 0, "ns_gemm launch failed: ", cudaGetErrorString(static_cast<cudaError_t>(rc)));
}

// Answered once per device: the properties query costs milliseconds of host time, and the optimizers ask on every
// orthogonalisation (it made the distributed Muon step host-bound).
bool ns_supported() {
    static int cached[64];                     // 0 unknown, 1 yes, 2 no
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    if (dev >= 0 && dev < 64 && cached[dev] != 0) return cached[dev] == 1;
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return false;
    if (dev >= 0 && dev < 64) cached[dev] = major == 10 ? 1 : 2;
    return major == 10;
}

// one TN GEMM, exposed for tests and benchmarks: C = alpha * A @ B^T + beta * D, optional Ct = C^T
// symmetric: the caller asserts that alpha * A @ B^T + beta * D is symmetric (e.g. B is A); half the tiles are skipped
at::Tensor ns_gemm_tn(const at::Tensor& A, const at::Tensor& B, const c10::optional<at::Tensor>& D, double alpha, double beta,
                      bool want_transpose, bool symmetric, int64_t tile_n) {
    c10::cuda::CUDAGuard guard(A.device());
    at::Tensor a3 = A.dim() == 2 ? A.unsqueeze(0) : A;
    at::Tensor b3 = B.dim() == 2 ? B.unsqueeze(0) : B;
    c10::optional<at::Tensor> d3;
    if (D.has_value() && D->defined()) d3 = D->dim() == 2 ? D->unsqueeze(0) : *D;
    at::Tensor C = at::empty({a3.size(0), a3.size(1), b3.size(1)}, a3.options());
    at::Tensor err = at::zeros({1}, a3.options().dtype(at::kInt));
    c10::optional<at::Tensor> Ct;
    if (want_transpose) Ct = at::empty({a3.size(0), b3.size(1), a3.size(1)}, a3.options());
    TORCH_CHECK(!(symmetric && want_transpose), "a symmetric product is its own transpose");
    gemm(a3.contiguous(), b3.contiguous(), d3, C, Ct, static_cast<float>(alpha), static_cast<float>(beta), err, symmetric,
         static_cast<int>(tile_n));
    TORCH_CHECK(err.item<int>() == 0, "ns_gemm: a bounded wait expired (code ", err.item<int>(), ")");
    if (want_transpose) return at::stack({C.reshape(-1), Ct->reshape(-1)});
    return A.dim() == 2 ? C.squeeze(0) : C;
}

// X: [batch, m, n] (or [m, n]) bf16, m <= n, already normalised.  coeffs: a, b, c per iteration.
// err: optional int32 device word that collects the kernels' wait-expired codes; when given, the call does not
// synchronise with the host and the caller reads the word when it wants to (one sync for many calls).
at::Tensor ns_iterate(const at::Tensor& X_in, const std::vector<double>& coeffs, const c10::optional<at::Tensor>& err_in) {
    TORCH_CHECK(coeffs.size() % 3 == 0 && !coeffs.empty(), "coefficients come in triples");
    TORCH_CHECK(X_in.is_cuda() && X_in.scalar_type() == at::kBFloat16, "bf16 CUDA input expected");
    c10::cuda::CUDAGuard guard(X_in.device());
    at::Tensor X = (X_in.dim() == 2 ? X_in.unsqueeze(0) : X_in).contiguous();
    const int64_t batch = X.size(0), m = X.size(1), n = X.size(2);
    TORCH_CHECK(m % 128 == 0 && n % 128 == 0, "ns_iterate: dimensions must be multiples of 128");
    at::Tensor Y = X.transpose(1, 2).contiguous();            // [batch, n, m]
    at::Tensor A = at::empty({batch, m, m}, X.options());
    at::Tensor B = at::empty({batch, m, m}, X.options());
    at::Tensor X2 = at::empty_like(X);
    at::Tensor Y2 = at::empty_like(Y);
    const bool own_err = !(err_in.has_value() && err_in->defined());
    at::Tensor err = own_err ? at::zeros({1}, X.options().dtype(at::kInt)) : *err_in;
    TORCH_CHECK(err.device() == X.device() && err.scalar_type() == at::kInt && err.numel() >= 1, "err: int32 tensor on the input's device");
    const size_t steps = coeffs.size() / 3;
    for (size_t s = 0; s < steps; ++s) {
        const float a = static_cast<float>(coeffs[3 * s]), b = static_cast<float>(coeffs[3 * s + 1]), c = static_cast<float>(coeffs[3 * s + 2]);
        gemm(X, X, c10::nullopt, A, c10::nullopt, 1.0f, 0.0f, err, true);      // A = X X^T        (symmetric)
        gemm(A, A, A, B, c10::nullopt, c, b, err, true);                        // B = b A + c A A  (symmetric)
        const bool last = (s + 1 == steps);
        gemm(B, Y, X, X2, last ? c10::optional<at::Tensor>() : c10::optional<at::Tensor>(Y2), 1.0f, a, err);   // X' = a X + B X
        std::swap(X, X2);
        if (!last) std::swap(Y, Y2);
    }
    if (own_err)
        TORCH_CHECK(err.item<int>() == 0, "ns_iterate: a bounded wait expired inside the GEMM kernel (code ", err.item<int>(), ")");
    return X_in.dim() == 2 ? X.squeeze(0) : X;
}

// Whole orthogonalisation of G [batch, r, c] (or [r, c]) bf16 with dimensions that are multiples of 128:
// Frobenius normalisation (fp32 accumulation), scale + transpose in one pass, the iteration, and the result
// written straight into `out` (same shape as G; may be G itself) - no separate divide, transpose or copy pass.
at::Tensor ns_orthogonalize(const at::Tensor& G_in, const std::vector<double>& coeffs, double eps,
                            const c10::optional<at::Tensor>& out_in, const c10::optional<at::Tensor>& err_in) {
    TORCH_CHECK(coeffs.size() % 3 == 0 && !coeffs.empty(), "coefficients come in triples");
    TORCH_CHECK(G_in.is_cuda() && G_in.scalar_type() == at::kBFloat16 && G_in.is_contiguous(), "contiguous bf16 CUDA input expected");
    c10::cuda::CUDAGuard guard(G_in.device());
    at::Tensor G = G_in.dim() == 2 ? G_in.unsqueeze(0) : G_in;
    TORCH_CHECK(G.dim() == 3, "expected [rows, cols] or [batch, rows, cols]");
    const int64_t batch = G.size(0), r = G.size(1), c = G.size(2);
    TORCH_CHECK(r % 128 == 0 && c % 128 == 0, "ns_orthogonalize: dimensions must be multiples of 128");
    at::Tensor out = (out_in.has_value() && out_in->defined()) ? (out_in->dim() == 2 ? out_in->unsqueeze(0) : *out_in)
                                                               : at::empty_like(G);
    TORCH_CHECK(out.sizes() == G.sizes() && out.is_contiguous() && out.scalar_type() == at::kBFloat16 && out.device() == G.device(),
                "out must match the input");
    const bool own_err = !(err_in.has_value() && err_in->defined());
    at::Tensor err = own_err ? at::zeros({1}, G.options().dtype(at::kInt)) : *err_in;
    cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();

    at::Tensor norms = at::linalg_vector_norm(G, 2, at::IntArrayRef({1, 2}), false, at::kFloat);     // [batch], fp32 accumulate
    at::Tensor inv = (norms + eps).reciprocal();
    at::Tensor Xs = at::empty_like(G);                          // [batch, r, c]
    at::Tensor XsT = at::empty({batch, c, r}, G.options());     // [batch, c, r]
    int rc = apexb_ns_prep(G.data_ptr(), inv.data_ptr<float>(), Xs.data_ptr(), XsT.data_ptr(), static_cast<int>(batch),
                           static_cast<int>(r), static_cast<int>(c), stream);
    TORCH_CHECK(rc == 0, "ns_prep launch failed: ", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    const bool tall = r > c;
    at::Tensor X = tall ? XsT : Xs;                             // [batch, m, n], m <= n
    at::Tensor Y = tall ? Xs : XsT;                             // [batch, n, m]
    const int64_t m = X.size(1);
    at::Tensor A = at::empty({batch, m, m}, G.options());
    at::Tensor B = at::empty({batch, m, m}, G.options());
    at::Tensor X2 = at::empty_like(X);
    at::Tensor Y2 = at::empty_like(Y);
    const size_t steps = coeffs.size() / 3;
    for (size_t s = 0; s < steps; ++s) {
        const float a = static_cast<float>(coeffs[3 * s]), b = static_cast<float>(coeffs[3 * s + 1]), cc = static_cast<float>(coeffs[3 * s + 2]);
        gemm(X, X, c10::nullopt, A, c10::nullopt, 1.0f, 0.0f, err, true);      // A = X X^T        (symmetric)
        gemm(A, A, A, B, c10::nullopt, cc, b, err, true);                       // B = b A + c A A  (symmetric)
        const bool last = (s + 1 == steps);
        if (!last) {
            gemm(B, Y, X, X2, c10::optional<at::Tensor>(Y2), 1.0f, a, err);     // X' = a X + B X, Y' = X'^T
            std::swap(X, X2);
            std::swap(Y, Y2);
        } else if (tall) {
            gemm(B, Y, X, X2, c10::optional<at::Tensor>(out), 1.0f, a, err);    // the result in G's orientation is Y'
        } else {
            gemm(B, Y, X, out, c10::nullopt, 1.0f, a, err);
        }
    }
    if (own_err)
        TORCH_CHECK(err.item<int>() == 0, "ns_orthogonalize: a bounded wait expired inside the GEMM kernel (code ", err.item<int>(), ")");
    return G_in.dim() == 2 ? out.squeeze(0) : out;
}

}  // namespace

void register_ns(pybind11::module_& m) {
    m.def("ns_orthogonalize", &ns_orthogonalize, pybind11::arg("G"), pybind11::arg("coeffs"), pybind11::arg("eps") = 1e-7,
          pybind11::arg("out") = pybind11::none(), pybind11::arg("err") = pybind11::none());
    m.def("ns_supported", &ns_supported);
    m.def("ns_iterate", &ns_iterate, pybind11::arg("X"), pybind11::arg("coeffs"), pybind11::arg("err") = pybind11::none());
    m.def("ns_gemm_tn", &ns_gemm_tn, pybind11::arg("A"), pybind11::arg("B"), pybind11::arg("D"), pybind11::arg("alpha"),
          pybind11::arg("beta"), pybind11::arg("want_transpose"), pybind11::arg("symmetric") = false,
          pybind11::arg("tile_n") = 0);
}

// Python bindings and host-side runtime of the native library.
//
// StatePlan is the resident launch plan of the fused optimizer-state kernels: a
// device array of segment descriptors built once per parameter group, patched
// in place when gradient pointers move, and launched with a handful of scalars
// per step.  It replaces the reference's per-step metadata upload through
// constant memory (apexw/csrc/apexw_cuda_kernel.cu:488-496) and its per-step
// Python list building (apexw/optimizer.py:406-1341).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cstring>
#include <vector>
#include "api.h"
#include "state_plan.h"

using apexb_host::StatePlan;

void register_model_ops(pybind11::module_& m);
void register_symm(pybind11::module_& m);
void register_muon(pybind11::module_& m);
void register_ns(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.attr("abi_version") = 1;
    m.attr("chunk_elems") = apexb::kChunk2048;
    pybind11::class_<StatePlan>(m, "StatePlan")
        .def(pybind11::init<int, std::vector<at::Tensor>, std::vector<at::Tensor>, std::vector<at::Tensor>,
                            std::vector<at::Tensor>, std::vector<at::Tensor>, std::vector<int64_t>, std::vector<int64_t>,
                            std::vector<int64_t>, std::vector<int64_t>, int64_t, std::vector<std::vector<int64_t>>>(),
             pybind11::arg("kernel_class"), pybind11::arg("params"), pybind11::arg("m"), pybind11::arg("v"),
             pybind11::arg("m_scale"), pybind11::arg("v_scale"), pybind11::arg("flags"), pybind11::arg("salts"),
             pybind11::arg("block_sizes"), pybind11::arg("offsets") = std::vector<int64_t>(), pybind11::arg("device_index") = -1,
             pybind11::arg("decay_ranges") = std::vector<std::vector<int64_t>>())
        .def_property_readonly("mixed_decay_chunks", &StatePlan::mixed_decay_chunks)
        .def_property_readonly("kernel_class", &StatePlan::kernel_class)
        .def("step", &StatePlan::step, pybind11::call_guard<pybind11::gil_scoped_release>(),
             pybind11::arg("grads"), pybind11::arg("beta1"), pybind11::arg("beta2"), pybind11::arg("step_size"), pybind11::arg("eps_scaled"),
             pybind11::arg("eps"), pybind11::arg("eps_quad"), pybind11::arg("eps_quad_scaled"), pybind11::arg("decay_factor"),
             pybind11::arg("inv_scale"), pybind11::arg("gain_hi"), pybind11::arg("gain_lo"), pybind11::arg("step_key"), pybind11::arg("flags"),
             pybind11::arg("found_inf"), pybind11::arg("grad_scale"), pybind11::arg("ctas_per_sm"), pybind11::arg("beta3") = 0.0,
             pybind11::arg("slow_ratio") = 0.0, pybind11::arg("lr") = 0.0)
        .def("step_zero", &StatePlan::step_zero, pybind11::call_guard<pybind11::gil_scoped_release>(),
             pybind11::arg("peer_grad"), pybind11::arg("peer_param"), pybind11::arg("peer_signal"), pybind11::arg("rank"),
             pybind11::arg("epoch"), pybind11::arg("timeout_ms"), pybind11::arg("status"), pybind11::arg("grad_dtype_code"),
             pybind11::arg("param_dtype_code"), pybind11::arg("beta1"), pybind11::arg("beta2"), pybind11::arg("step_size"),
             pybind11::arg("eps_scaled"), pybind11::arg("eps"), pybind11::arg("eps_quad"), pybind11::arg("eps_quad_scaled"),
             pybind11::arg("decay_factor"), pybind11::arg("inv_scale"), pybind11::arg("gain_hi"), pybind11::arg("gain_lo"),
             pybind11::arg("step_key"), pybind11::arg("flags"), pybind11::arg("mc_grad") = 0, pybind11::arg("mc_param") = 0,
             pybind11::arg("clip_total_sq") = c10::optional<at::Tensor>(), pybind11::arg("clip_max_norm") = 0.0)
        .def("reduce_zero", &StatePlan::reduce_zero, pybind11::call_guard<pybind11::gil_scoped_release>())
        .def("set_device_scalars", &StatePlan::set_device_scalars, pybind11::arg("step_dev"), pybind11::arg("lr_dev"),
             pybind11::arg("step_host"), pybind11::arg("lr_host"), pybind11::arg("alpha"), pybind11::arg("weight_decay"), pybind11::arg("seed"))
        .def("clear_device_scalars", &StatePlan::clear_device_scalars)
        .def("set_cta_cap", &StatePlan::set_cta_cap)
        .def("set_v_scale_log4", &StatePlan::set_v_scale_log4)
        .def_property_readonly("total_chunks", &StatePlan::total_chunks)
        .def_property_readonly("num_segments", &StatePlan::num_segments)
        .def_property_readonly("launches", &StatePlan::launches);
    m.def("table_fault_report", &apexb_host::table_fault_report, pybind11::arg("clear") = true,
          "Debug mode: {code, segment, chunk, skipped} of the single-GPU kernels, then of the peer kernels (synchronises)");
    m.def("table_check_selftest", &apexb_host::table_check_selftest, "Bit mask of the table checker's self-test cases that behaved");
    m.def("zero_norm_exchange", &apexb_host::zero_norm_exchange, pybind11::call_guard<pybind11::gil_scoped_release>());
    register_model_ops(m);
    register_symm(m);
    register_muon(m);
    register_ns(m);
}

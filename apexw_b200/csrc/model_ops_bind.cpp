// Python bindings of the model-side fused ops (model_ops.cu).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "api.h"

namespace {

void ok(int err, const char* what) {
    TORCH_CHECK(err == 0, what, " failed: ", cudaGetErrorString(static_cast<cudaError_t>(err)));
}

int bf16_flag(const at::Tensor& t) {
    TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kFloat, "expected bf16 or fp32 tensor");
    return t.scalar_type() == at::kBFloat16 ? 1 : 0;
}

void check_vec(const at::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.is_contiguous(), name, " must be a contiguous CUDA tensor");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, " must be 16-byte aligned");
}

int sms(const at::Tensor& t) { return at::cuda::getDeviceProperties(t.device().index())->multiProcessorCount; }

std::tuple<at::Tensor, at::Tensor, at::Tensor> rmsnorm_fwd(const at::Tensor& x, const c10::optional<at::Tensor>& residual,
                                                           const at::Tensor& weight, double eps) {
    check_vec(x, "x");
    TORCH_CHECK(x.dim() == 2, "x must be (rows, H)");
    const int rows = static_cast<int>(x.size(0)), H = static_cast<int>(x.size(1));
    at::Tensor w = weight.scalar_type() == x.scalar_type() ? weight.contiguous() : weight.to(x.scalar_type()).contiguous();
    check_vec(w, "weight");
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor y = at::empty_like(x);
    at::Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
    at::Tensor h = x;
    const void* res = nullptr;
    if (residual.has_value() && residual->defined()) {
        check_vec(*residual, "residual");
        TORCH_CHECK(residual->sizes() == x.sizes() && residual->scalar_type() == x.scalar_type(), "residual must match x");
        h = at::empty_like(x);
        res = residual->data_ptr();
    }
    ok(apexb_rmsnorm_fwd(x.data_ptr(), res, w.data_ptr(), y.data_ptr(), h.data_ptr(), rstd.data_ptr<float>(), rows, H,
                         static_cast<float>(eps), bf16_flag(x), sms(x), at::cuda::getCurrentCUDAStream().stream()),
       "rmsnorm_fwd");
    return {y, h, rstd};
}

std::tuple<at::Tensor, at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const c10::optional<at::Tensor>& dres, const at::Tensor& h,
                                               const at::Tensor& weight, const at::Tensor& rstd) {
    check_vec(dy, "dy");
    check_vec(h, "h");
    const int rows = static_cast<int>(h.size(0)), H = static_cast<int>(h.size(1));
    at::Tensor w = weight.scalar_type() == h.scalar_type() ? weight.contiguous() : weight.to(h.scalar_type()).contiguous();
    c10::cuda::CUDAGuard guard(h.device());
    at::Tensor dx = at::empty_like(h);
    at::Tensor dw = at::empty({H}, h.options().dtype(at::kFloat));
    const int nparts = apexb_rmsnorm_bwd_parts(rows, sms(h));
    at::Tensor partial = at::empty({nparts, H}, h.options().dtype(at::kFloat));   // scratch: per-CTA weight-gradient partials
    const void* dr = nullptr;
    if (dres.has_value() && dres->defined()) {
        check_vec(*dres, "dres");
        dr = dres->data_ptr();
    }
    ok(apexb_rmsnorm_bwd(dy.data_ptr(), dr, h.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(),
                         dw.data_ptr<float>(), partial.data_ptr<float>(), nparts, rows, H, bf16_flag(h),
                         at::cuda::getCurrentCUDAStream().stream()),
       "rmsnorm_bwd");
    return {dx, dw};
}

at::Tensor swiglu_fwd(const at::Tensor& gu) {
    check_vec(gu, "gu");
    const int64_t F = gu.size(-1) / 2;
    const int64_t rows = gu.numel() / (2 * F);
    auto shape = gu.sizes().vec();
    shape.back() = F;
    c10::cuda::CUDAGuard guard(gu.device());
    at::Tensor y = at::empty(shape, gu.options());
    ok(apexb_swiglu_fwd(gu.data_ptr(), y.data_ptr(), rows, static_cast<int>(F), bf16_flag(gu), sms(gu),
                        at::cuda::getCurrentCUDAStream().stream()), "swiglu_fwd");
    return y;
}

at::Tensor swiglu_bwd(const at::Tensor& dy, const at::Tensor& gu) {
    check_vec(gu, "gu");
    check_vec(dy, "dy");
    const int64_t F = gu.size(-1) / 2;
    const int64_t rows = gu.numel() / (2 * F);
    c10::cuda::CUDAGuard guard(gu.device());
    at::Tensor dgu = at::empty_like(gu);
    ok(apexb_swiglu_bwd(dy.data_ptr(), gu.data_ptr(), dgu.data_ptr(), rows, static_cast<int>(F), bf16_flag(gu), sms(gu),
                        at::cuda::getCurrentCUDAStream().stream()), "swiglu_bwd");
    return dgu;
}

at::Tensor rope_apply(const at::Tensor& qkv, const at::Tensor& cosv, const at::Tensor& sinv, int64_t n_rot, bool inverse) {
    check_vec(qkv, "qkv");
    TORCH_CHECK(qkv.dim() == 4, "qkv must be (B, S, heads, D)");
    TORCH_CHECK(cosv.scalar_type() == at::kFloat && sinv.scalar_type() == at::kFloat && cosv.is_contiguous() && sinv.is_contiguous(),
                "cos/sin tables must be contiguous fp32");
    const int64_t S = qkv.size(1), heads = qkv.size(2), D = qkv.size(3);
    TORCH_CHECK(cosv.size(0) >= S && cosv.size(1) == D / 2, "cos/sin tables too small");
    c10::cuda::CUDAGuard guard(qkv.device());
    at::Tensor out = at::empty_like(qkv);
    // the table's row stride is D/2, so positions index it directly; tokens wrap every S
    ok(apexb_rope(qkv.data_ptr(), out.data_ptr(), cosv.data_ptr<float>(), sinv.data_ptr<float>(), qkv.size(0) * S,
                  static_cast<int>(S), static_cast<int>(heads), static_cast<int>(D), static_cast<int>(n_rot), inverse ? 1 : 0,
                  bf16_flag(qkv), sms(qkv), at::cuda::getCurrentCUDAStream().stream()), "rope");
    return out;
}

at::Tensor cross_entropy_fwd_bwd(at::Tensor logits, const at::Tensor& targets, double scale,
                                 c10::optional<at::Tensor> scale_dev) {
    check_vec(logits, "logits");
    TORCH_CHECK(logits.dim() == 2 && targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.is_cuda(),
                "logits (rows, V) and int64 CUDA targets expected");
    TORCH_CHECK(targets.numel() == logits.size(0), "one target per row");
    const float* sd = nullptr;
    if (scale_dev.has_value() && scale_dev->defined()) {
        TORCH_CHECK(scale_dev->device() == logits.device() && scale_dev->scalar_type() == at::kFloat && scale_dev->numel() == 1,
                    "scale_dev must be one fp32 value on the logits' device");
        sd = scale_dev->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(logits.device());
    at::Tensor losses = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
    ok(apexb_cross_entropy(logits.data_ptr(), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()), losses.data_ptr<float>(),
                           static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)), static_cast<float>(scale), sd,
                           bf16_flag(logits), at::cuda::getCurrentCUDAStream().stream()), "cross_entropy");
    return losses;
}

}  // namespace

void register_model_ops(pybind11::module_& m) {
    m.def("rmsnorm_fwd", &rmsnorm_fwd);
    m.def("rmsnorm_bwd", &rmsnorm_bwd);
    m.def("swiglu_fwd", &swiglu_fwd);
    m.def("swiglu_bwd", &swiglu_bwd);
    m.def("rope_apply", &rope_apply);
    m.def("cross_entropy_fwd_bwd", &cross_entropy_fwd_bwd, pybind11::arg("logits"), pybind11::arg("targets"), pybind11::arg("scale"),
          pybind11::arg("scale_dev") = c10::optional<at::Tensor>());
}

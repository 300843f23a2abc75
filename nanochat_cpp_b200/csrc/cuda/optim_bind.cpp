// Tensor-level wrappers of the optimizer kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "optim.h"

namespace {

using torch::Tensor;
inline cudaStream_t cur() { return at::cuda::getCurrentCUDAStream(); }
inline __nv_bfloat16* bptr(const Tensor& t) { return reinterpret_cast<__nv_bfloat16*>(t.data_ptr()); }

void adamw_update(Tensor& master, const c10::optional<Tensor>& value, const Tensor& grad, Tensor& m, Tensor& v,
                  double lr, double beta1, double beta2, double eps, double weight_decay, int64_t step,
                  const c10::optional<Tensor>& grad_scale) {
  TORCH_CHECK(master.is_cuda() && master.is_contiguous() && grad.is_contiguous() && m.is_contiguous() &&
                  v.is_contiguous(),
              "adamw: contiguous CUDA tensors expected");
  TORCH_CHECK(master.scalar_type() == torch::kFloat32 && grad.scalar_type() == torch::kFloat32, "adamw: fp32 state");
  const c10::cuda::CUDAGuard g(master.device());
  __nv_bfloat16* vp = nullptr;
  if (value.has_value()) {
    TORCH_CHECK(value->scalar_type() == torch::kBFloat16 && value->is_contiguous(), "adamw: bf16 compute copy");
    vp = bptr(*value);
  }
  nc::adamw_update(master.data_ptr<float>(), vp, grad.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                   master.numel(), lr, beta1, beta2, eps, weight_decay, step,
                   grad_scale.has_value() ? grad_scale->data_ptr<float>() : nullptr, cur());
}

void muon_nesterov(const Tensor& grad, Tensor& buf1, Tensor& x, Tensor& row_sumsq, double momentum,
                   const c10::optional<Tensor>& grad_scale) {
  const c10::cuda::CUDAGuard g(grad.device());
  TORCH_CHECK(grad.dim() == 2 && grad.is_contiguous() && buf1.is_contiguous() && x.is_contiguous(), "muon_nesterov");
  nc::muon_nesterov(grad.data_ptr<float>(), buf1.data_ptr<float>(), x.data_ptr<float>(), row_sumsq.data_ptr<float>(),
                    grad.size(0), grad.size(1), momentum,
                    grad_scale.has_value() ? grad_scale->data_ptr<float>() : nullptr, cur());
}
void muon_scale_rows(const Tensor& x, const Tensor& row_scale, const Tensor& all_scale, Tensor& out) {
  const c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && out.is_contiguous(), "muon_scale_rows");
  nc::muon_scale_rows(x.data_ptr<float>(), row_scale.data_ptr<float>(), all_scale.data_ptr<float>(), bptr(out),
                      x.size(0), x.size(1), cur());
}
void muon_apply(Tensor& master, const c10::optional<Tensor>& value, const Tensor& xb, const Tensor& scale0,
                const Tensor& line_scale, bool lines_are_rows, double lr, double wd) {
  const c10::cuda::CUDAGuard g(master.device());
  TORCH_CHECK(master.dim() == 2 && master.is_contiguous() && xb.is_contiguous(), "muon_apply");
  nc::muon_apply(master.data_ptr<float>(), value.has_value() ? bptr(*value) : nullptr, bptr(xb),
                 scale0.data_ptr<float>(), line_scale.data_ptr<float>(), lines_are_rows, master.size(0),
                 master.size(1), lr, wd, cur());
}
Tensor relu2(const Tensor& x) {
  const c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(x.is_contiguous() && x.scalar_type() == torch::kBFloat16, "relu2: contiguous bf16");
  Tensor y = torch::empty_like(x);
  nc::relu2_bf16(bptr(x), bptr(y), x.numel(), cur());
  return y;
}
void cast_f32_bf16(const Tensor& x, Tensor& y) {
  const c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && x.numel() == y.numel(), "cast");
  nc::cast_f32_bf16(x.data_ptr<float>(), bptr(y), x.numel(), cur());
}

}  // namespace

void register_optim(pybind11::module_& m) {
  m.def("adamw_update", &adamw_update);
  m.def("muon_nesterov_batched", [](const Tensor& grad_ptrs, const Tensor& buf1_ptrs, Tensor& x, Tensor& row_ss,
                                    double momentum, const c10::optional<Tensor>& grad_scale) {
    const c10::cuda::CUDAGuard g(x.device());
    TORCH_CHECK(x.dim() == 3 && x.is_contiguous() && x.size(2) % 8 == 0 && grad_ptrs.scalar_type() == torch::kInt64 &&
                    grad_ptrs.numel() == x.size(0) && buf1_ptrs.numel() == x.size(0), "muon_nesterov_batched");
    nc::muon_nesterov_batched(reinterpret_cast<const long long*>(grad_ptrs.data_ptr<int64_t>()),
                              reinterpret_cast<const long long*>(buf1_ptrs.data_ptr<int64_t>()), x.data_ptr<float>(),
                              row_ss.data_ptr<float>(), x.size(0), x.size(1), x.size(2), momentum,
                              grad_scale.has_value() ? grad_scale->data_ptr<float>() : nullptr,
                              at::cuda::getCurrentCUDAStream());
  });
  m.def("muon_scale_rows_batched", [](const Tensor& x, const Tensor& row_scale, const Tensor& all_scale, Tensor& out) {
    const c10::cuda::CUDAGuard g(x.device());
    TORCH_CHECK(x.dim() == 3 && x.is_contiguous() && out.is_contiguous() && row_scale.is_contiguous() &&
                    all_scale.is_contiguous() && x.size(2) % 8 == 0, "muon_scale_rows_batched");
    nc::muon_scale_rows_batched(x.data_ptr<float>(), row_scale.data_ptr<float>(), all_scale.data_ptr<float>(), bptr(out),
                                x.size(0), x.size(1), x.size(2), at::cuda::getCurrentCUDAStream());
  });
  m.def("muon_line_sumsq", [](const Tensor& x, bool reduce_cols) {
    const c10::cuda::CUDAGuard g(x.device());
    TORCH_CHECK(x.dim() == 3 && x.is_contiguous() && x.scalar_type() == torch::kBFloat16 && x.size(2) % 8 == 0,
                "muon_line_sumsq");
    Tensor out = torch::empty({x.size(0), reduce_cols ? x.size(1) : x.size(2)}, x.options().dtype(torch::kFloat32));
    nc::muon_line_sumsq(bptr(x), out.data_ptr<float>(), x.size(0), x.size(1), x.size(2), reduce_cols,
                        at::cuda::getCurrentCUDAStream());
    return out;
  });
  m.def("muon_apply_batched", [](const Tensor& master_ptrs, const c10::optional<Tensor>& value_ptrs, const Tensor& xb,
                                 const Tensor& scale0, const Tensor& line_scale, bool lines_are_rows, double lr,
                                 double wd) {
    const c10::cuda::CUDAGuard g(xb.device());
    TORCH_CHECK(xb.dim() == 3 && xb.is_contiguous() && scale0.is_contiguous() && line_scale.is_contiguous() &&
                    master_ptrs.numel() == xb.size(0), "muon_apply_batched");
    nc::muon_apply_batched(reinterpret_cast<const long long*>(master_ptrs.data_ptr<int64_t>()),
                           value_ptrs.has_value() ? reinterpret_cast<const long long*>(value_ptrs->data_ptr<int64_t>())
                                                  : nullptr,
                           bptr(xb), scale0.data_ptr<float>(), line_scale.data_ptr<float>(), lines_are_rows, xb.size(0),
                           xb.size(1), xb.size(2), lr, wd, at::cuda::getCurrentCUDAStream());
  });
  m.def("muon_prescale", [](const Tensor& row_ss, Tensor& row_scale, Tensor& all_scale) {
    const c10::cuda::CUDAGuard g(row_ss.device());
    TORCH_CHECK(row_ss.dim() == 2 && row_ss.is_contiguous() && row_scale.is_contiguous() && all_scale.is_contiguous() &&
                    row_scale.numel() == row_ss.numel() && all_scale.numel() == row_ss.size(0), "muon_prescale");
    nc::muon_prescale(row_ss.data_ptr<float>(), row_scale.data_ptr<float>(), all_scale.data_ptr<float>(),
                      row_ss.size(0), row_ss.size(1), at::cuda::getCurrentCUDAStream());
  });
  m.def("muon_poststats", [](const Tensor& line_ss, const Tensor& buf2_ptrs, Tensor& scale, Tensor& line_scale,
                             int64_t line_len, double target_norm, double beta2) {
    const c10::cuda::CUDAGuard g(line_ss.device());
    TORCH_CHECK(line_ss.dim() == 2 && line_ss.is_contiguous() && line_scale.is_contiguous() &&
                    line_scale.numel() == line_ss.numel() && scale.numel() == line_ss.size(0) &&
                    buf2_ptrs.scalar_type() == torch::kInt64 && buf2_ptrs.numel() == line_ss.size(0), "muon_poststats");
    nc::muon_poststats(line_ss.data_ptr<float>(), reinterpret_cast<const long long*>(buf2_ptrs.data_ptr<int64_t>()),
                       scale.data_ptr<float>(), line_scale.data_ptr<float>(), line_ss.size(0), line_ss.size(1), line_len,
                       target_norm, beta2, at::cuda::getCurrentCUDAStream());
  });
  m.def("muon_tiny", [](const Tensor& grad_ptrs, const Tensor& buf1_ptrs, const Tensor& buf2_ptrs,
                        const Tensor& master_ptrs, const c10::optional<Tensor>& value_ptrs, int64_t rows, int64_t cols,
                        double momentum, double beta2, double lr, double wd, int64_t ns_steps,
                        const c10::optional<Tensor>& grad_scale, const std::vector<std::vector<double>>& coeffs) {
    const c10::cuda::CUDAGuard g(grad_ptrs.device());
    const int64_t P = grad_ptrs.numel();
    for (const Tensor* t : {&grad_ptrs, &buf1_ptrs, &buf2_ptrs, &master_ptrs})
      TORCH_CHECK(t->scalar_type() == torch::kInt64 && t->is_contiguous() && t->numel() == P && t->is_cuda(),
                  "muon_tiny: pointer tables are int64 device tensors of one length");
    TORCH_CHECK(!value_ptrs.has_value() || (value_ptrs->scalar_type() == torch::kInt64 && value_ptrs->numel() == P),
                "muon_tiny: value table");
    TORCH_CHECK(coeffs.size() == 5, "muon_tiny: five coefficient triples");
    double c[5][3];
    for (int i = 0; i < 5; ++i) {
      TORCH_CHECK(coeffs[i].size() == 3, "muon_tiny: five coefficient triples");
      for (int j = 0; j < 3; ++j) c[i][j] = coeffs[i][j];
    }
    auto tab = [](const Tensor& t) { return reinterpret_cast<const long long*>(t.data_ptr<int64_t>()); };
    const char* err = nc::muon_tiny(tab(grad_ptrs), tab(buf1_ptrs), tab(buf2_ptrs), tab(master_ptrs),
                                    value_ptrs.has_value() ? tab(*value_ptrs) : nullptr, static_cast<int>(P),
                                    static_cast<int>(rows), static_cast<int>(cols), static_cast<float>(momentum),
                                    static_cast<float>(beta2), static_cast<float>(lr), static_cast<float>(wd),
                                    static_cast<int>(ns_steps),
                                    grad_scale.has_value() ? grad_scale->data_ptr<float>() : nullptr, c,
                                    at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(err == nullptr, err);
  });
  m.def("muon_nesterov", &muon_nesterov);
  m.def("muon_scale_rows", &muon_scale_rows);
  m.def("muon_apply", &muon_apply);
  m.def("relu2", &relu2);
  m.def("cast_f32_bf16", &cast_f32_bf16);
}

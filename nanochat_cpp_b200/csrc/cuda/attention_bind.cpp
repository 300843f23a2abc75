// Tensor-level wrappers of the attention kernels. q/k/v/o/do and the gradients are [B, T, H, D]
// bf16 views with unit stride in D (they may be column slices of wider token-major buffers).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "attention.h"

namespace {

using torch::Tensor;

void chk4(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16, name, ": expected a CUDA bf16 tensor");
  TORCH_CHECK(t.dim() == 4 && t.stride(3) == 1, name, ": expected [B,T,H,D] with unit stride in D");
  TORCH_CHECK(t.stride(0) % 8 == 0 && t.stride(1) % 8 == 0 && t.stride(2) % 8 == 0, name,
              ": strides must be multiples of 8 elements");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name, ": base address must be 16-byte aligned");
}

void fill_common(nc::AttnArgs& a, const Tensor& q, const Tensor& k, const Tensor& v, int64_t window_left, double scale,
                 int64_t q_offset) {
  chk4(q, "q");
  chk4(k, "k");
  chk4(v, "v");
  a.B = q.size(0), a.Tq = q.size(1), a.H = q.size(2), a.D = q.size(3);
  a.Tk = k.size(1), a.KVH = k.size(2);
  TORCH_CHECK(k.size(0) == a.B && v.size(0) == a.B && v.size(1) == a.Tk && v.size(2) == a.KVH && k.size(3) == a.D &&
                  v.size(3) == a.D,
              "attention: q/k/v shapes disagree");
  a.q_offset = static_cast<int>(q_offset < 0 ? a.Tk - a.Tq : q_offset);
  a.window_left = static_cast<int>(window_left);
  a.scale = static_cast<float>(scale);
  a.Q = q.data_ptr(), a.K = k.data_ptr(), a.V = v.data_ptr();
  a.q_stride_b = q.stride(0), a.q_stride_t = q.stride(1), a.q_stride_h = q.stride(2);
  a.k_stride_b = k.stride(0), a.k_stride_t = k.stride(1), a.k_stride_h = k.stride(2);
  a.v_stride_b = v.stride(0), a.v_stride_t = v.stride(1), a.v_stride_h = v.stride(2);
}

std::vector<Tensor> attention_fwd(const Tensor& q, const Tensor& k, const Tensor& v, int64_t window_left, double scale,
                                  int64_t q_offset, Tensor status, int64_t variant) {
  const c10::cuda::CUDAGuard guard(q.device());
  nc::AttnArgs a;
  fill_common(a, q, k, v, window_left, scale, q_offset);
  Tensor o = torch::empty({a.B, a.Tq, a.H, a.D}, q.options());
  Tensor lse = torch::empty({a.B, a.H, a.Tq}, q.options().dtype(torch::kFloat32));
  a.O = o.data_ptr();
  a.o_stride_b = o.stride(0), a.o_stride_t = o.stride(1), a.o_stride_h = o.stride(2);
  a.lse = lse.data_ptr<float>();
  a.status = status.data_ptr<int>();
  const char* err = variant == 1 ? nc::attention_fwd(a, at::cuda::getCurrentCUDAStream())
                                 : nc::attention_fwd2(a, at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(err == nullptr, err);
  return {o, lse};
}

void attention_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& lse,
                   const Tensor& d_o, Tensor& dq, Tensor& dk, Tensor& dv, int64_t window_left, double scale,
                   int64_t q_offset, Tensor status, const c10::optional<Tensor>& ds_scratch) {
  const c10::cuda::CUDAGuard guard(q.device());
  nc::AttnArgs a;
  fill_common(a, q, k, v, window_left, scale, q_offset);
  chk4(o, "o");
  chk4(d_o, "do");
  chk4(dq, "dq");
  chk4(dk, "dk");
  chk4(dv, "dv");
  TORCH_CHECK(lse.is_contiguous() && lse.scalar_type() == torch::kFloat32, "lse must be contiguous fp32");
  TORCH_CHECK(dq.sizes() == q.sizes() && dk.sizes() == k.sizes() && dv.sizes() == v.sizes(), "gradient shapes");
  Tensor delta = torch::empty_like(lse);
  a.O = o.data_ptr();
  a.o_stride_b = o.stride(0), a.o_stride_t = o.stride(1), a.o_stride_h = o.stride(2);
  a.lse = lse.data_ptr<float>();
  a.dO = d_o.data_ptr();
  a.do_stride_b = d_o.stride(0), a.do_stride_t = d_o.stride(1), a.do_stride_h = d_o.stride(2);
  a.delta = delta.data_ptr<float>();
  a.dQ = dq.data_ptr(), a.dK = dk.data_ptr(), a.dV = dv.data_ptr();
  a.dq_stride_b = dq.stride(0), a.dq_stride_t = dq.stride(1), a.dq_stride_h = dq.stride(2);
  a.dk_stride_b = dk.stride(0), a.dk_stride_t = dk.stride(1), a.dk_stride_h = dk.stride(2);
  a.dv_stride_b = dv.stride(0), a.dv_stride_t = dv.stride(1), a.dv_stride_h = dv.stride(2);
  a.status = status.data_ptr<int>();
  if (ds_scratch.has_value()) {
    // [B, H, Tk padded to 128, Tq padded to 128] bf16, contiguous
    const Tensor& ds = *ds_scratch;
    TORCH_CHECK(ds.dim() == 4 && ds.is_contiguous() && ds.scalar_type() == torch::kBFloat16 && ds.size(0) == a.B &&
                    ds.size(1) == a.H && ds.size(2) % 128 == 0 && ds.size(3) % 128 == 0 && ds.size(2) >= a.Tk &&
                    ds.size(3) >= a.Tq,
                "ds_scratch must be a contiguous bf16 [B, H, Tk128, Tq128] tensor");
    a.dS = ds.data_ptr();
    a.ds_tk = ds.size(2), a.ds_tq = ds.size(3);
  }
  const char* err = nc::attention_bwd(a, at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(err == nullptr, err);
}

}  // namespace

void register_attention(pybind11::module_& m) {
  m.def("attention_fwd", &attention_fwd);
  m.def("attention_bwd", &attention_bwd, pybind11::arg("q"), pybind11::arg("k"), pybind11::arg("v"), pybind11::arg("o"),
        pybind11::arg("lse"), pybind11::arg("d_o"), pybind11::arg("dq"), pybind11::arg("dk"), pybind11::arg("dv"),
        pybind11::arg("window_left"), pybind11::arg("scale"), pybind11::arg("q_offset"), pybind11::arg("status"),
        pybind11::arg("ds_scratch") = c10::optional<Tensor>());
}

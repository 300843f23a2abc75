// Tensor-level wrappers of the row kernels (rowops.cu). Shapes and dtypes are checked here; the
// launchers only see pointers.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "rowops.h"

namespace ncbind {
int* device_status(int device);   // bindings.cpp: the device's status word
}

namespace {
inline int* st(const torch::Tensor& like) { return ncbind::device_status(like.get_device()); }

using torch::Tensor;
using nc::bf16;

inline const bf16* bp(const Tensor& t) { return reinterpret_cast<const bf16*>(t.data_ptr()); }
inline bf16* bpm(Tensor& t) { return reinterpret_cast<bf16*>(t.data_ptr()); }
inline cudaStream_t cur() { return at::cuda::getCurrentCUDAStream(); }

void chk(const Tensor& t, c10::ScalarType dt, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, ": expected a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == dt, name, ": unexpected dtype ", t.scalar_type());
}
void chk_rows(const Tensor& t, const char* name) {
  chk(t, torch::kBFloat16, name);
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, name, ": expected [rows, dim] with unit inner stride");
}
Tensor f32_empty(const Tensor& like, std::vector<int64_t> shape) {
  return torch::empty(shape, like.options().dtype(torch::kFloat32));
}
Tensor f32_zeros(const Tensor& like, std::vector<int64_t> shape) {
  return torch::zeros(shape, like.options().dtype(torch::kFloat32));
}

std::vector<Tensor> rmsnorm_fwd(const Tensor& x, double eps) {
  chk_rows(x, "x");
  const c10::cuda::CUDAGuard g(x.device());
  Tensor y = torch::empty({x.size(0), x.size(1)}, x.options());
  Tensor rstd = f32_empty(x, {x.size(0)});
  nc::rmsnorm_fwd(bp(x), x.stride(0), bpm(y), rstd.data_ptr<float>(), x.size(0), x.size(1), eps, cur());
  return {y, rstd};
}
// MXFP8 companions: the same kernels also emit the output as E4M3 codes + scale atoms (128-row tiles).
bool mx_ok(const Tensor& x) {
  return x.size(1) % 128 == 0 && x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0;
}
Tensor mx_atoms(const Tensor& x) {
  const int64_t tiles = (x.size(0) + 127) / 128;
  return torch::empty({tiles * (x.size(1) / 128) * 512}, x.options().dtype(torch::kUInt8));
}
std::vector<Tensor> rmsnorm_fwd_mx(const Tensor& x, double eps) {
  chk_rows(x, "x");
  TORCH_CHECK(mx_ok(x), "rmsnorm_fwd_mx: dim % 128 == 0 and 16-byte aligned rows");
  const c10::cuda::CUDAGuard g(x.device());
  Tensor y = torch::empty({x.size(0), x.size(1)}, x.options());
  Tensor rstd = f32_empty(x, {x.size(0)});
  Tensor yq = torch::empty({x.size(0), x.size(1)}, x.options().dtype(torch::kUInt8));
  Tensor sf = mx_atoms(x);
  nc::rmsnorm_fwd(bp(x), x.stride(0), bpm(y), rstd.data_ptr<float>(), x.size(0), x.size(1), eps, cur(),
                  yq.data_ptr<uint8_t>(), sf.data_ptr<uint8_t>());
  return {y, rstd, yq, sf};
}
std::vector<Tensor> blend_norm_fwd_mx(const Tensor& x, const Tensor& x0, const Tensor& lam_r, const Tensor& lam_0,
                                      double eps) {
  chk_rows(x, "x");
  chk_rows(x0, "x0");
  chk(lam_r, torch::kFloat32, "lam_r");
  chk(lam_0, torch::kFloat32, "lam_0");
  TORCH_CHECK(x.is_contiguous() && x0.is_contiguous() && x.sizes() == x0.sizes() && mx_ok(x) && mx_ok(x0),
              "blend_mx: bad inputs");
  const c10::cuda::CUDAGuard g(x.device());
  Tensor xr = torch::empty_like(x), h = torch::empty_like(x);
  Tensor rstd = f32_empty(x, {x.size(0)});
  Tensor hq = torch::empty({x.size(0), x.size(1)}, x.options().dtype(torch::kUInt8));
  Tensor sf = mx_atoms(x);
  nc::blend_norm_fwd(bp(x), bp(x0), lam_r.data_ptr<float>(), lam_0.data_ptr<float>(), bpm(xr), bpm(h),
                     rstd.data_ptr<float>(), x.size(0), x.size(1), eps, cur(), hq.data_ptr<uint8_t>(),
                     sf.data_ptr<uint8_t>());
  return {xr, h, rstd, hq, sf};
}

Tensor rmsnorm_apply(const Tensor& x, const Tensor& rstd) {
  chk_rows(x, "x");
  chk(rstd, torch::kFloat32, "rstd");
  const c10::cuda::CUDAGuard g(x.device());
  Tensor y = torch::empty({x.size(0), x.size(1)}, x.options());
  nc::rmsnorm_apply(bp(x), x.stride(0), rstd.data_ptr<float>(), bpm(y), x.size(0), x.size(1), cur());
  return y;
}
Tensor rmsnorm_bwd(const Tensor& x, const Tensor& dy, const Tensor& rstd, const c10::optional<Tensor>& residual) {
  chk_rows(x, "x");
  chk_rows(dy, "dy");
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous(), "rmsnorm_bwd: contiguous inputs expected");
  if (residual.has_value()) TORCH_CHECK(residual->is_contiguous() && residual->sizes() == x.sizes(), "bad residual");
  const c10::cuda::CUDAGuard g(x.device());
  Tensor dx = torch::empty_like(x);
  nc::rmsnorm_bwd(bp(x), bp(dy), rstd.data_ptr<float>(), residual.has_value() ? bp(*residual) : nullptr, bpm(dx),
                  x.size(0), x.size(1), cur());
  return dx;
}
std::vector<Tensor> blend_norm_fwd(const Tensor& x, const Tensor& x0, const Tensor& lam_r, const Tensor& lam_0,
                                   double eps) {
  chk_rows(x, "x");
  chk_rows(x0, "x0");
  chk(lam_r, torch::kFloat32, "lam_r");
  chk(lam_0, torch::kFloat32, "lam_0");
  TORCH_CHECK(x.is_contiguous() && x0.is_contiguous() && x.sizes() == x0.sizes(), "blend: bad inputs");
  const c10::cuda::CUDAGuard g(x.device());
  Tensor xr = torch::empty_like(x), h = torch::empty_like(x);
  Tensor rstd = f32_empty(x, {x.size(0)});
  nc::blend_norm_fwd(bp(x), bp(x0), lam_r.data_ptr<float>(), lam_0.data_ptr<float>(), bpm(xr), bpm(h),
                     rstd.data_ptr<float>(), x.size(0), x.size(1), eps, cur());
  return {xr, h, rstd};
}
// Returns (dx, dlam[2]); dx0 is updated in place (overwritten when !accumulate).
std::vector<Tensor> blend_bwd(const Tensor& dxr, const Tensor& x, const Tensor& x0, const Tensor& lam_r,
                              const Tensor& lam_0, Tensor& dx0, bool accumulate) {
  chk_rows(dxr, "dxr");
  TORCH_CHECK(dxr.is_contiguous() && x.is_contiguous() && x0.is_contiguous() && dx0.is_contiguous(), "blend_bwd");
  const c10::cuda::CUDAGuard g(x.device());
  Tensor dx = torch::empty_like(x);
  Tensor dlam = f32_zeros(x, {2});
  nc::blend_bwd(bp(dxr), bp(x), bp(x0), lam_r.data_ptr<float>(), lam_0.data_ptr<float>(), bpm(dx), bpm(dx0),
                accumulate, dlam.data_ptr<float>(), x.numel(), cur());
  return {dx, dlam};
}
// dx0 is written (or accumulated into); g_lam_r / g_lam_0 are one-element fp32 views of the gradient buffer.
Tensor norm_blend_bwd(const Tensor& xr, const Tensor& dh, const Tensor& rstd, const Tensor& residual,
                      const c10::optional<Tensor>& extra, const Tensor& x, const Tensor& x0, const Tensor& lam_r,
                      const Tensor& lam_0, Tensor& dx0, bool accumulate, Tensor& g_lam_r, Tensor& g_lam_0) {
  chk_rows(xr, "xr");
  chk_rows(dh, "dh");
  chk(rstd, torch::kFloat32, "rstd");
  chk(g_lam_r, torch::kFloat32, "g_lam_r");
  chk(g_lam_0, torch::kFloat32, "g_lam_0");
  TORCH_CHECK(xr.is_contiguous() && dh.is_contiguous() && residual.is_contiguous() && x.is_contiguous() &&
                  x0.is_contiguous() && dx0.is_contiguous() && dh.sizes() == xr.sizes() && residual.sizes() == xr.sizes() &&
                  x.numel() == xr.numel() && x0.numel() == xr.numel() && dx0.numel() == xr.numel() &&
                  rstd.numel() == xr.size(0) && g_lam_r.numel() == 1 && g_lam_0.numel() == 1,
              "norm_blend_bwd: shapes");
  const c10::cuda::CUDAGuard g(xr.device());
  const float* ex = nullptr;
  int ex_cols = 0;
  if (extra.has_value()) {
    chk(*extra, torch::kFloat32, "extra");
    TORCH_CHECK(extra->is_contiguous() && extra->dim() == 2 && extra->size(0) == xr.size(0), "norm_blend_bwd: extra");
    ex = extra->data_ptr<float>();
    ex_cols = extra->size(1);
  }
  Tensor dx = torch::empty_like(xr);
  const char* err = nc::norm_blend_bwd(bp(xr), bp(dh), rstd.data_ptr<float>(), bp(residual), ex, ex_cols, bp(x), bp(x0),
                                       lam_r.data_ptr<float>(), lam_0.data_ptr<float>(), bpm(dx), bpm(dx0), accumulate,
                                       g_lam_r.data_ptr<float>(), g_lam_0.data_ptr<float>(), xr.size(0), xr.size(1), cur());
  TORCH_CHECK(err == nullptr, err);
  return dx;
}
Tensor backout_fwd(const Tensor& x, const Tensor& xb, const Tensor& lam) {
  TORCH_CHECK(x.is_contiguous() && xb.is_contiguous(), "backout_fwd");
  const c10::cuda::CUDAGuard g(x.device());
  Tensor y = torch::empty_like(x);
  nc::backout_fwd(bp(x), bp(xb), lam.data_ptr<float>(), bpm(y), x.numel(), cur());
  return y;
}
std::vector<Tensor> backout_bwd(const Tensor& dy, const Tensor& xb, const Tensor& lam) {
  TORCH_CHECK(dy.is_contiguous() && xb.is_contiguous(), "backout_bwd");
  const c10::cuda::CUDAGuard g(dy.device());
  Tensor dxb = torch::empty_like(dy);
  Tensor dlam = f32_zeros(dy, {1});
  nc::backout_bwd(bp(dy), bp(xb), lam.data_ptr<float>(), bpm(dxb), dlam.data_ptr<float>(), dy.numel(), cur());
  return {dxb, dlam};
}
Tensor add(const Tensor& a, const Tensor& b) {
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && a.sizes() == b.sizes(), "add");
  const c10::cuda::CUDAGuard g(a.device());
  Tensor o = torch::empty_like(a);
  nc::add_bf16(bp(a), bp(b), bpm(o), a.numel(), cur());
  return o;
}
void add_cols(Tensor& dh, const Tensor& extra) {
  chk_rows(dh, "dh");
  chk(extra, torch::kFloat32, "extra");
  TORCH_CHECK(extra.is_contiguous() && extra.size(0) == dh.size(0), "add_cols");
  const c10::cuda::CUDAGuard g(dh.device());
  nc::add_cols(bpm(dh), dh.stride(0), extra.data_ptr<float>(), dh.size(0), extra.size(1), cur());
}

// x: [B, T, H, D] view whose (T, H, D) strides are (ld, D, 1) and B stride T*ld.
void chk_heads(const Tensor& t, const char* name) {
  chk(t, torch::kBFloat16, name);
  TORCH_CHECK(t.dim() == 4 && t.stride(3) == 1 && t.stride(2) == t.size(3) && t.stride(0) == t.size(1) * t.stride(1),
              name, ": expected a [B,T,H,D] view of token rows");
}
Tensor qk_prep_fwd_one(const Tensor& x, const Tensor& cos, const Tensor& sin, const c10::optional<Tensor>& positions,
                       double eps, double scale) {
  chk_heads(x, "x");
  chk(cos, torch::kFloat32, "cos");
  const c10::cuda::CUDAGuard g(x.device());
  const int B = x.size(0), T = x.size(1), H = x.size(2), D = x.size(3);
  Tensor y = torch::empty({B, T, H, D}, x.options());
  const int* pos = nullptr;
  if (positions.has_value()) {
    chk(*positions, torch::kInt32, "positions");
    pos = positions->data_ptr<int>();
  }
  nc::qk_prep_fwd(bp(x), x.stride(1), bpm(y), static_cast<long long>(H) * D, cos.data_ptr<float>(),
                  sin.data_ptr<float>(), pos, B * T, T, H, D, eps, scale, cur());
  return y;
}
// out may be a column slice of a wider gradient buffer ([B,T,H,D] view).
void qk_prep_bwd_one(const Tensor& pre, const Tensor& grad, Tensor& out, const Tensor& cos, const Tensor& sin,
                     double eps, double scale) {
  chk_heads(pre, "pre");
  chk_heads(grad, "grad");
  chk_heads(out, "out");
  const c10::cuda::CUDAGuard g(pre.device());
  const int B = pre.size(0), T = pre.size(1), H = pre.size(2), D = pre.size(3);
  nc::qk_prep_bwd(bp(pre), pre.stride(1), bp(grad), grad.stride(1), bpm(out), out.stride(1), cos.data_ptr<float>(),
                  sin.data_ptr<float>(), B * T, T, H, D, eps, scale, cur());
}

Tensor value_gate_fwd(const Tensor& h, const Tensor& ve, const Tensor& gate_w, Tensor& v, int64_t D) {
  chk_rows(h, "h");
  chk_rows(v, "v");
  TORCH_CHECK(ve.is_contiguous() && gate_w.is_contiguous(), "value_gate_fwd");
  const c10::cuda::CUDAGuard g(h.device());
  const int KV = gate_w.size(0);
  Tensor gate = torch::empty({h.size(0), KV}, h.options());
  nc::value_gate_fwd(bp(h), h.stride(0), bp(ve), bp(gate_w), bpm(v), v.stride(0), bpm(gate), h.size(0), KV, D, cur());
  return gate;
}
// Same with the value-embedding rows gathered inside the kernel: table [vocab, KV * D], ids int32 [tokens].
Tensor value_gate_fwd_gather(const Tensor& h, const Tensor& ids, const Tensor& table, const Tensor& gate_w, Tensor& v,
                             int64_t D) {
  chk_rows(h, "h");
  chk_rows(v, "v");
  TORCH_CHECK(table.is_contiguous() && gate_w.is_contiguous() && table.scalar_type() == torch::kBFloat16 &&
                  ids.scalar_type() == torch::kInt32 && ids.is_contiguous() && ids.numel() == h.size(0),
              "value_gate_fwd_gather");
  const c10::cuda::CUDAGuard g(h.device());
  const int KV = gate_w.size(0);
  TORCH_CHECK(table.size(1) == KV * D, "value_gate_fwd_gather: table width");
  Tensor gate = torch::empty({h.size(0), KV}, h.options());
  nc::value_gate_fwd(bp(h), h.stride(0), bp(table), bp(gate_w), bpm(v), v.stride(0), bpm(gate), h.size(0), KV, D, cur(),
                     ids.data_ptr<int>(), table.size(0), st(h));
  return gate;
}
std::vector<Tensor> value_gate_bwd(const Tensor& h, const Tensor& ve, const Tensor& gate_w, const Tensor& gate,
                                   const Tensor& dv, int64_t D) {
  chk_rows(h, "h");
  chk_rows(dv, "dv");
  const c10::cuda::CUDAGuard g(h.device());
  const int KV = gate_w.size(0);
  Tensor dve = torch::empty({h.size(0), KV * D}, h.options());
  Tensor dh12 = f32_empty(h, {h.size(0), 12});
  Tensor dgw = f32_zeros(h, {KV, 12});
  nc::value_gate_bwd(bp(h), h.stride(0), bp(ve), bp(gate_w), bp(gate), bp(dv), dv.stride(0), bpm(dve),
                     dh12.data_ptr<float>(), dgw.data_ptr<float>(), h.size(0), KV, D, cur());
  return {dve, dh12, dgw};
}

std::vector<Tensor> smear_fwd(const Tensor& emb, const Tensor& gate_w, const Tensor& lam, int64_t seq,
                              const c10::optional<Tensor>& prev) {
  chk_rows(emb, "emb");
  TORCH_CHECK(emb.is_contiguous(), "smear_fwd");
  const c10::cuda::CUDAGuard g(emb.device());
  Tensor x0 = torch::empty_like(emb);
  Tensor sig = f32_empty(emb, {emb.size(0)});
  nc::smear_fwd(bp(emb), bp(gate_w), lam.data_ptr<float>(), prev.has_value() ? bp(*prev) : nullptr, bpm(x0),
                sig.data_ptr<float>(), emb.size(0), seq, emb.size(1), cur());
  return {x0, sig};
}
std::vector<Tensor> smear_bwd(const Tensor& emb, const Tensor& gate_w, const Tensor& lam, const Tensor& sig,
                              const Tensor& dx0, int64_t seq) {
  chk_rows(emb, "emb");
  TORCH_CHECK(emb.is_contiguous() && dx0.is_contiguous(), "smear_bwd");
  const c10::cuda::CUDAGuard g(emb.device());
  Tensor de = torch::empty_like(emb);
  Tensor dgw = f32_zeros(emb, {24});
  Tensor dlam = f32_zeros(emb, {1});
  nc::smear_bwd(bp(emb), bp(gate_w), lam.data_ptr<float>(), sig.data_ptr<float>(), bp(dx0), bpm(de),
                dgw.data_ptr<float>(), dlam.data_ptr<float>(), emb.size(0), seq, emb.size(1), cur());
  return {de, dgw, dlam};
}

Tensor embedding_fwd(const Tensor& ids, const Tensor& table) {
  chk(ids, torch::kInt32, "ids");
  chk_rows(table, "table");
  TORCH_CHECK(table.is_contiguous() && ids.is_contiguous(), "embedding_fwd");
  const c10::cuda::CUDAGuard g(table.device());
  Tensor out = torch::empty({ids.numel(), table.size(1)}, table.options());
  nc::embedding_fwd(ids.data_ptr<int>(), bp(table), bpm(out), ids.numel(), table.size(1), cur(), table.size(0),
                    st(table));
  return out;
}
void embedding_bwd(const Tensor& ids, const Tensor& dout, Tensor& dtable) {
  chk(ids, torch::kInt32, "ids");
  chk_rows(dout, "dout");
  chk(dtable, torch::kFloat32, "dtable");
  TORCH_CHECK(dtable.is_contiguous(), "embedding_bwd");
  const c10::cuda::CUDAGuard g(dout.device());
  nc::embedding_bwd(ids.data_ptr<int>(), bp(dout), dout.stride(0), dtable.data_ptr<float>(), ids.numel(),
                    dtable.size(1), cur(), dtable.size(0), st(dout));
}
void embedding_bwd_sorted(const Tensor& sorted_ids, const Tensor& perm, const Tensor& dout, Tensor& dtable) {
  chk(sorted_ids, torch::kInt32, "sorted_ids");
  chk(perm, torch::kInt32, "perm");
  chk_rows(dout, "dout");
  chk(dtable, torch::kFloat32, "dtable");
  TORCH_CHECK(dtable.is_contiguous() && sorted_ids.is_contiguous() && perm.is_contiguous() &&
                  perm.numel() == sorted_ids.numel() && dout.size(0) == sorted_ids.numel(),
              "embedding_bwd_sorted");
  const c10::cuda::CUDAGuard g(dout.device());
  nc::embedding_bwd_sorted(sorted_ids.data_ptr<int>(), perm.data_ptr<int>(), bp(dout), dout.stride(0),
                           dtable.data_ptr<float>(), sorted_ids.numel(), dtable.size(1), cur(), dtable.size(0),
                           st(dout));
}

// In place: `logits` becomes dlogits when want_grad. Returns per-row losses.
Tensor classifier_fwd_bwd(Tensor& logits, const Tensor& targets, int64_t vocab, const c10::optional<Tensor>& dscale,
                          const c10::optional<Tensor>& row_scale, double softcap, int64_t ignore_index,
                          bool want_grad) {
  chk_rows(logits, "logits");
  chk(targets, torch::kInt32, "targets");
  const c10::cuda::CUDAGuard g(logits.device());
  Tensor losses = f32_empty(logits, {logits.size(0)});
  const float* ds = nullptr;
  if (want_grad) {
    TORCH_CHECK(dscale.has_value(), "classifier: dlogit_scale required for the backward");
    chk(*dscale, torch::kFloat32, "dlogit_scale");
    ds = dscale->data_ptr<float>();
  }
  const float* rs = nullptr;
  if (row_scale.has_value()) {
    chk(*row_scale, torch::kFloat32, "row_scale");
    rs = row_scale->data_ptr<float>();
  }
  nc::classifier_fwd_bwd(bpm(logits), logits.stride(0), targets.data_ptr<int>(), losses.data_ptr<float>(), rs, ds,
                         logits.size(0), vocab, logits.size(1), softcap, ignore_index, want_grad, cur(),
                         st(logits));
  return losses;
}

// norm_clip[0] = ||g||, norm_clip[1] = min(1, clip/||g||) over a flat fp32 buffer.
Tensor grad_norm_clip(const Tensor& flat, double clip) {
  chk(flat, torch::kFloat32, "grad");
  TORCH_CHECK(flat.is_contiguous(), "grad_norm_clip");
  const c10::cuda::CUDAGuard g(flat.device());
  Tensor acc = torch::zeros({1}, flat.options().dtype(torch::kFloat64));
  Tensor out = f32_empty(flat, {2});
  nc::sumsq_f32(flat.data_ptr<float>(), flat.numel(), acc.data_ptr<double>(), cur());
  nc::finish_norm(acc.data_ptr<double>(), clip, out.data_ptr<float>(), cur());
  return out;
}
void sumsq_into(const Tensor& flat, Tensor& acc) {
  chk(flat, torch::kFloat32, "grad");
  chk(acc, torch::kFloat64, "acc");
  const c10::cuda::CUDAGuard g(flat.device());
  nc::sumsq_f32(flat.data_ptr<float>(), flat.numel(), acc.data_ptr<double>(), cur());
}

}  // namespace

void register_rowops(pybind11::module_& m) {
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_apply", &rmsnorm_apply);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("blend_norm_fwd", &blend_norm_fwd);
  m.def("rmsnorm_fwd_mx", &rmsnorm_fwd_mx);
  m.def("blend_norm_fwd_mx", &blend_norm_fwd_mx);
  m.def("blend_bwd", &blend_bwd);
  m.def("backout_fwd", &backout_fwd);
  m.def("backout_bwd", &backout_bwd);
  m.def("add", &add);
  m.def("add_cols", &add_cols);
  m.def("qk_prep_fwd_one", &qk_prep_fwd_one);
  m.def("qk_prep_bwd_one", &qk_prep_bwd_one);
  m.def("value_gate_fwd", &value_gate_fwd);
  m.def("value_gate_bwd", &value_gate_bwd);
  m.def("value_gate_fwd_gather", &value_gate_fwd_gather);
  m.def("smear_fwd", &smear_fwd);
  m.def("smear_bwd", &smear_bwd);
  m.def("norm_blend_bwd", &norm_blend_bwd);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("embedding_bwd_sorted", &embedding_bwd_sorted);
  m.def("classifier_fwd_bwd", &classifier_fwd_bwd);
  m.def("grad_norm_clip", &grad_norm_clip);
  m.def("sumsq_into", &sumsq_into);
}

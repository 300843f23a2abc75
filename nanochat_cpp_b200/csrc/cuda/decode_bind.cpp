// Tensor-level wrappers of the paged-KV inference kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "decode.h"

namespace ncbind {
int* device_status(int device);   // bindings.cpp: the device's status word
}
#include "pdl_launch.h"

namespace {

using torch::Tensor;
inline __nv_bfloat16* bp(const Tensor& t) { return reinterpret_cast<__nv_bfloat16*>(t.data_ptr()); }

// k_new / v_new: [B, T, KV, D] views with row (token) stride ld and contiguous [KV, D] rows.
void kv_append(Tensor& k_pool, Tensor& v_pool, const Tensor& page_table, const Tensor& positions, const Tensor& k_new,
               const Tensor& v_new) {
  const c10::cuda::CUDAGuard g(k_pool.device());
  TORCH_CHECK(k_pool.is_contiguous() && v_pool.is_contiguous() && k_pool.dim() == 4, "pools must be [P, page, KV, D]");
  TORCH_CHECK(page_table.scalar_type() == torch::kInt32 && page_table.is_contiguous(), "page_table must be int32");
  TORCH_CHECK(positions.scalar_type() == torch::kInt32 && positions.is_contiguous() && positions.dim() == 2,
              "positions must be int32 [B, T]");
  TORCH_CHECK(k_new.dim() == 4 && k_new.stride(3) == 1 && k_new.stride(2) == k_new.size(3) &&
                  k_new.stride(0) == k_new.size(1) * k_new.stride(1),
              "k_new must be a [B,T,KV,D] view of token rows");
  TORCH_CHECK(v_new.dim() == 4 && v_new.stride(3) == 1 && v_new.stride(2) == v_new.size(3) &&
                  v_new.stride(0) == v_new.size(1) * v_new.stride(1),
              "v_new must be a [B,T,KV,D] view of token rows");
  const int row = k_pool.size(2) * k_pool.size(3);
  TORCH_CHECK(row % 8 == 0 && k_new.stride(1) % 8 == 0 && v_new.stride(1) % 8 == 0, "rows must allow 16-byte copies");
  nc::kv_append(bp(k_pool), bp(v_pool), page_table.data_ptr<int>(), page_table.size(1), positions.data_ptr<int>(),
                bp(k_new), k_new.stride(1), bp(v_new), v_new.stride(1), positions.size(0), positions.size(1),
                k_pool.size(1), row, at::cuda::getCurrentCUDAStream(), k_pool.size(0),
                ncbind::device_status(k_pool.get_device()));
}

// qk: [B, >= (H + KV) * D] rows of the fused projection (q heads first), v: [B, KV * D] rows (any row stride);
// cos / sin: fp32 [positions, D / 2]; positions: int32 [B]. Returns q prepared, dense [B, H, D].
Tensor decode_prep_append(const Tensor& qk, const Tensor& v, const Tensor& cos, const Tensor& sin,
                          const Tensor& positions, Tensor& k_pool, Tensor& v_pool, const Tensor& page_table, int64_t H,
                          double eps, double scale) {
  const c10::cuda::CUDAGuard g(qk.device());
  TORCH_CHECK(k_pool.is_contiguous() && v_pool.is_contiguous() && k_pool.dim() == 4, "pools must be [P, page, KV, D]");
  const int KV = k_pool.size(2), D = k_pool.size(3), B = qk.size(0);
  TORCH_CHECK(qk.dim() == 2 && qk.scalar_type() == torch::kBFloat16 && qk.stride(1) == 1 && qk.size(1) >= (H + KV) * D,
              "qk must be bf16 rows holding the q and k heads");
  TORCH_CHECK(v.dim() == 2 && v.scalar_type() == torch::kBFloat16 && v.stride(1) == 1 && v.size(0) == B &&
                  v.size(1) == KV * D,
              "v must be bf16 [B, KV * D]");
  TORCH_CHECK(cos.scalar_type() == torch::kFloat32 && sin.scalar_type() == torch::kFloat32 && cos.is_contiguous() &&
                  sin.is_contiguous() && cos.size(-1) == D / 2,
              "cos / sin must be fp32 [positions, D / 2]");
  TORCH_CHECK(positions.scalar_type() == torch::kInt32 && positions.is_contiguous() && positions.numel() == B,
              "positions must be int32 [B]");
  TORCH_CHECK(page_table.scalar_type() == torch::kInt32 && page_table.is_contiguous() && page_table.size(0) == B,
              "page_table must be int32 [B, max_pages]");
  Tensor q_out = torch::empty({B, H, D}, qk.options());
  const char* err = nc::decode_prep_append(bp(qk), qk.stride(0), bp(v), v.stride(0), cos.data_ptr<float>(),
                                           sin.data_ptr<float>(), positions.data_ptr<int>(), page_table.data_ptr<int>(),
                                           page_table.size(1), k_pool.size(1), bp(q_out), bp(k_pool), bp(v_pool), B,
                                           static_cast<int>(H), KV, D, static_cast<float>(eps), static_cast<float>(scale),
                                           at::cuda::getCurrentCUDAStream(), k_pool.size(0),
                                           ncbind::device_status(k_pool.get_device()));
  TORCH_CHECK(err == nullptr, err);
  return q_out;
}

Tensor softcap_logits(const Tensor& logits, int64_t vocab, double cap) {
  const c10::cuda::CUDAGuard g(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.scalar_type() == torch::kBFloat16 && logits.stride(1) == 1 &&
                  vocab <= logits.size(1) && vocab % 2 == 0,
              "softcap_logits: bf16 [rows, >= vocab], even vocab");
  Tensor out = torch::empty({logits.size(0), vocab}, logits.options().dtype(torch::kFloat32));
  nc::softcap_logits(bp(logits), logits.stride(0), out.data_ptr<float>(), logits.size(0), static_cast<int>(vocab),
                     static_cast<float>(cap), at::cuda::getCurrentCUDAStream());
  return out;
}

Tensor argmax_rows(const Tensor& logits, int64_t vocab) {
  const c10::cuda::CUDAGuard g(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.scalar_type() == torch::kBFloat16 && logits.stride(1) == 1 &&
                  vocab <= logits.size(1) && vocab > 0,
              "argmax_rows: bf16 [rows, >= vocab]");
  Tensor out = torch::empty({logits.size(0)}, logits.options().dtype(torch::kInt64));
  nc::argmax_rows(bp(logits), logits.stride(0), reinterpret_cast<long long*>(out.data_ptr<int64_t>()), logits.size(0),
                  static_cast<int>(vocab), at::cuda::getCurrentCUDAStream());
  return out;
}

Tensor paged_decode_attention(const Tensor& q, const Tensor& k_pool, const Tensor& v_pool, const Tensor& page_table,
                              const Tensor& seq_lens, int64_t window_left, double scale) {
  const c10::cuda::CUDAGuard g(q.device());
  // q may be a slice of a wider row (the q half of the fused q/k preparation output): heads and channels dense
  TORCH_CHECK(q.dim() == 3 && q.scalar_type() == torch::kBFloat16 && q.stride(2) == 1 && q.stride(1) == q.size(2) &&
                  q.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(q.data_ptr()) & 15) == 0,
              "q must be bf16 [B, H, D] with dense heads and 16-byte aligned rows");
  TORCH_CHECK(seq_lens.scalar_type() == torch::kInt32 && seq_lens.is_contiguous(), "seq_lens must be int32");
  Tensor out = torch::empty({q.size(0), q.size(1), q.size(2)}, q.options());
  nc::DecodeArgs a;
  a.q_stride_b = q.stride(0);
  a.B = q.size(0), a.H = q.size(1), a.D = q.size(2), a.KV = k_pool.size(2);
  a.q = bp(q), a.k_pool = bp(k_pool), a.v_pool = bp(v_pool);
  a.page_table = page_table.data_ptr<int>();
  a.max_pages = page_table.size(1);
  a.page_size = k_pool.size(1);
  a.seq_lens = seq_lens.data_ptr<int>();
  a.window_left = static_cast<int>(window_left);
  a.scale = static_cast<float>(scale);
  a.out = bp(out);
  int max_keys = a.max_pages * a.page_size;
  if (window_left >= 0 && window_left + 1 < max_keys) max_keys = static_cast<int>(window_left) + 1;
  a.splits = nc::decode_splits(a.B, a.KV, max_keys);
  Tensor part_acc, part_ml;
  if (a.splits > 1) {
    const auto f32 = q.options().dtype(torch::kFloat32);
    part_acc = torch::empty({a.B, a.H, a.splits, a.D}, f32);
    part_ml = torch::empty({a.B, a.H, a.splits, 2}, f32);
    a.part_acc = part_acc.data_ptr<float>();
    a.part_ml = part_ml.data_ptr<float>();
  }
  const char* err = nc::paged_decode_attention(a, at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(err == nullptr, err);
  return out;
}

}  // namespace

void register_decode(pybind11::module_& m) {
  m.def("kv_append", &kv_append);
  m.def("decode_prep_append", &decode_prep_append);
  m.def("softcap_logits", &softcap_logits);
  m.def("argmax_rows", &argmax_rows);
  m.def("set_pdl_enabled", [](bool on) { nc::set_pdl_enabled(on); });
  m.def("pdl_enabled", []() { return nc::pdl_enabled(); });
  m.def("paged_decode_attention", &paged_decode_attention);
}

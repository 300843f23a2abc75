// Tensor-level wrappers of the paged-KV inference kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "decode.h"

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
                k_pool.size(1), row, at::cuda::getCurrentCUDAStream());
}

Tensor paged_decode_attention(const Tensor& q, const Tensor& k_pool, const Tensor& v_pool, const Tensor& page_table,
                              const Tensor& seq_lens, int64_t window_left, double scale) {
  const c10::cuda::CUDAGuard g(q.device());
  TORCH_CHECK(q.dim() == 3 && q.is_contiguous() && q.scalar_type() == torch::kBFloat16, "q must be bf16 [B, H, D]");
  TORCH_CHECK(seq_lens.scalar_type() == torch::kInt32 && seq_lens.is_contiguous(), "seq_lens must be int32");
  Tensor out = torch::empty_like(q);
  nc::DecodeArgs a;
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
  m.def("paged_decode_attention", &paged_decode_attention);
}

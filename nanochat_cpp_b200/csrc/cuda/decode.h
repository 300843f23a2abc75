// Host interface of the paged-KV inference kernels (decode.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace nc {

struct DecodeArgs {
  int B = 0, H = 0, KV = 0, D = 0;
  const __nv_bfloat16* q = nullptr;       // [B, H, D], prepared (normed, rotated, scaled)
  long long q_stride_b = 0;               // elements between sequences in q (0: H * D, contiguous); 16-byte multiples
  const __nv_bfloat16* k_pool = nullptr;  // [pages, page_size, KV, D]
  const __nv_bfloat16* v_pool = nullptr;
  const int* page_table = nullptr;        // [B, max_pages]
  int max_pages = 0, page_size = 16;
  const int* seq_lens = nullptr;          // [B], including the token being decoded
  int window_left = -1;
  float scale = 1.0f;
  __nv_bfloat16* out = nullptr;           // [B, H, D]
  // Key splits per (sequence, kv head). With splits > 1 the kernel needs scratch: part_acc [B, H, splits, D] and
  // part_ml [B, H, splits, 2] floats.
  int splits = 1;
  float* part_acc = nullptr;
  float* part_ml = nullptr;
};

// Key splits that fill the GPU for B sequences of at most `max_keys` attended keys.
int decode_splits(int B, int KV, int max_keys);

// Rows k_new / v_new ([B*T, row_elems], leading dimensions k_ld / v_ld) go to absolute positions positions[B*T]
// (negative = skip) of their sequence's pages. A position past the page table, a negative page, or (with
// `num_pages` > 0, the pool's size) a page outside the pool is not written and records code 7 in `status`.
void kv_append(__nv_bfloat16* k_pool, __nv_bfloat16* v_pool, const int* page_table, int max_pages,
               const int* positions, const __nv_bfloat16* k_new, long long k_ld, const __nv_bfloat16* v_new,
               long long v_ld, int B, int T, int page_size, int row_elems, cudaStream_t s, int num_pages = 0,
               int* status = nullptr);

// Decode prologue in one launch (head_dim 128): q / k heads of the fused row `qk` ([tokens, >= (H + KV) * D], q heads
// first) get head RMSNorm -> RoPE at positions[tok] -> scale; q goes to q_out [tokens, H, D], k and the value row
// v ([tokens, KV * D]) go into the token's page of the pools. One token per sequence (page_table row = token).
const char* decode_prep_append(const __nv_bfloat16* qk, long long ld_qk, const __nv_bfloat16* v, long long ld_v,
                               const float* cosT, const float* sinT, const int* positions, const int* page_table,
                               int max_pages, int page_size, __nv_bfloat16* q_out, __nv_bfloat16* k_pool,
                               __nv_bfloat16* v_pool, int tokens, int H, int KV, int D, float eps, float scale,
                               cudaStream_t s, int num_pages = 0, int* status = nullptr);

// out fp32 [rows, vocab] = cap * tanh(logits[:, :vocab] / cap); logits bf16 rows with leading dimension ld; vocab even.
void softcap_logits(const __nv_bfloat16* logits, long long ld, float* out, int rows, int vocab, float cap, cudaStream_t s);

// out[r] = argmax over logits[r, 0 .. vocab) (lowest index among equal values); logits bf16 rows, leading dimension ld.
void argmax_rows(const __nv_bfloat16* logits, long long ld, long long* out, int rows, int vocab, cudaStream_t s);

const char* paged_decode_attention(const DecodeArgs& args, cudaStream_t s);

}  // namespace nc

// Inference kernels for the paged KV cache: append new keys / values into 16-token pages, and single-query
// attention over the pages (one query token per sequence, GQA, causal + left window).
//
// The reference decodes one row at a time over a contiguous cache and runs the attention through batched
// cuBLAS products (src/generate.cc:266-412, backends/cuda/kernels/attention_dispatch.h:38-48). Decode attention
// is bandwidth-bound (every cached key and value is read once per step), so this kernel streams K and V pages
// with 16-byte loads and keeps the online softmax in fp32 registers: one CTA per (sequence, kv head), the query
// heads of the group share the K / V traffic.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "decode.h"

namespace nc {

namespace {

__global__ void __launch_bounds__(256) kv_append_kernel(__nv_bfloat16* __restrict__ k_pool,
                                                        __nv_bfloat16* __restrict__ v_pool,
                                                        const int* __restrict__ page_table, int max_pages,
                                                        const int* __restrict__ positions,
                                                        const __nv_bfloat16* __restrict__ k_new, long long k_ld,
                                                        const __nv_bfloat16* __restrict__ v_new, long long v_ld,
                                                        int tokens_per_seq, int total_tokens, int page_size,
                                                        int row_elems) {
  const int tok = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= total_tokens) return;
  const int lane = threadIdx.x & 31;
  const int pos = positions[tok];
  if (pos < 0) return;
  const int b = tok / tokens_per_seq;
  const int page = page_table[b * max_pages + pos / page_size];
  const long long dst = (static_cast<long long>(page) * page_size + pos % page_size) * row_elems;
  const uint4* ks = reinterpret_cast<const uint4*>(k_new + static_cast<long long>(tok) * k_ld);
  const uint4* vs = reinterpret_cast<const uint4*>(v_new + static_cast<long long>(tok) * v_ld);
  uint4* kd = reinterpret_cast<uint4*>(k_pool + dst);
  uint4* vd = reinterpret_cast<uint4*>(v_pool + dst);
  for (int i = lane; i < row_elems / 8; i += 32) {
    kd[i] = ks[i];
    vd[i] = vs[i];
  }
}

constexpr int kChunk = 64;  // keys per step

// grid (KV heads, B); block = D threads (one output dimension per thread); the group's heads loop inside.
template <int D, int G>
__global__ void __launch_bounds__(D) paged_decode_kernel(const __nv_bfloat16* __restrict__ q,  // [B, H, D]
                                                         const __nv_bfloat16* __restrict__ k_pool,
                                                         const __nv_bfloat16* __restrict__ v_pool,
                                                         const int* __restrict__ page_table, int max_pages,
                                                         const int* __restrict__ seq_lens, int H, int KV,
                                                         int page_size, int window_left, float scale_log2,
                                                         __nv_bfloat16* __restrict__ out) {
  __shared__ float q_s[G][D];
  __shared__ float p_s[G][kChunk];
  __shared__ __nv_bfloat16 k_s[kChunk][D + 8];  // +8 keeps rows 16-byte aligned and off the same bank
  const int kvh = blockIdx.x, b = blockIdx.y;
  const int t = threadIdx.x;
  const int len = seq_lens[b];
  if (len <= 0) return;
  const int qpos = len - 1;
  const int first = window_left >= 0 ? max(0, qpos - window_left) : 0;
  for (int g = 0; g < G; ++g)
    q_s[g][t] = __bfloat162float(q[(static_cast<long long>(b) * H + kvh * G + g) * D + t]) * scale_log2;
  float m[G], l[G], acc[G];
#pragma unroll
  for (int g = 0; g < G; ++g) m[g] = -CUDART_INF_F, l[g] = 0.0f, acc[g] = 0.0f;
  const long long row = static_cast<long long>(KV) * D;  // elements per (page slot)
  for (int c0 = (first / kChunk) * kChunk; c0 <= qpos; c0 += kChunk) {
    __syncthreads();
    // stage the K chunk: thread t copies 16-byte pieces of key rows
    for (int i = t; i < kChunk * (D / 8); i += D) {
      const int j = i / (D / 8), part = i % (D / 8);
      const int key = c0 + j;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (key <= qpos) {
        const int page = page_table[b * max_pages + key / page_size];
        v = *reinterpret_cast<const uint4*>(k_pool + (static_cast<long long>(page) * page_size + key % page_size) * row +
                                            kvh * D + part * 8);
      }
      *reinterpret_cast<uint4*>(&k_s[j][part * 8]) = v;
    }
    __syncthreads();
    // scores: thread t < kChunk handles key c0 + t for every head of the group
    if (t < kChunk) {
      const int key = c0 + t;
      const bool ok = key <= qpos && key >= first;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = 0.0f;
#pragma unroll 8
        for (int d = 0; d < D; ++d) s += q_s[g][d] * __bfloat162float(k_s[t][d]);
        p_s[g][t] = ok ? s : -CUDART_INF_F;
      }
    }
    __syncthreads();
    // online softmax (every thread recomputes the chunk statistics: 64 values) and the V accumulation
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float cm = m[g];
      for (int j = 0; j < kChunk; ++j) cm = fmaxf(cm, p_s[g][j]);
      const float alpha = m[g] == -CUDART_INF_F ? 0.0f : exp2f(m[g] - cm);
      float a = acc[g] * alpha, ls = l[g] * alpha;
      for (int j = 0; j < kChunk; ++j) {
        const int key = c0 + j;
        if (key > qpos) break;
        const float pj = exp2f(p_s[g][j] - cm);
        if (pj == 0.0f) continue;
        const int page = page_table[b * max_pages + key / page_size];
        const float vv = __bfloat162float(
            v_pool[(static_cast<long long>(page) * page_size + key % page_size) * row + kvh * D + t]);
        a += pj * vv;
        ls += pj;
      }
      acc[g] = a, l[g] = ls, m[g] = cm;
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g)
    out[(static_cast<long long>(b) * H + kvh * G + g) * D + t] = __float2bfloat16_rn(acc[g] / l[g]);
}

template <int D>
const char* launch_decode(const DecodeArgs& a, cudaStream_t s) {
  const dim3 grid(a.KV, a.B);
  const int G = a.H / a.KV;
  const float sl2 = a.scale * 1.4426950408889634f;
#define NC_DECODE(GV)                                                                                          \
  paged_decode_kernel<D, GV><<<grid, D, 0, s>>>(a.q, a.k_pool, a.v_pool, a.page_table, a.max_pages, a.seq_lens, \
                                                a.H, a.KV, a.page_size, a.window_left, sl2, a.out)
  switch (G) {
    case 1: NC_DECODE(1); break;
    case 2: NC_DECODE(2); break;
    case 4: NC_DECODE(4); break;
    case 8: NC_DECODE(8); break;
    default: return "paged_decode_attention: group size must be 1, 2, 4 or 8";
  }
#undef NC_DECODE
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace

void kv_append(__nv_bfloat16* k_pool, __nv_bfloat16* v_pool, const int* page_table, int max_pages,
               const int* positions, const __nv_bfloat16* k_new, long long k_ld, const __nv_bfloat16* v_new,
               long long v_ld, int B, int T, int page_size, int row_elems, cudaStream_t s) {
  const int total = B * T;
  if (total <= 0) return;
  kv_append_kernel<<<(total + 7) / 8, 256, 0, s>>>(k_pool, v_pool, page_table, max_pages, positions, k_new, k_ld,
                                                   v_new, v_ld, T, total, page_size, row_elems);
}

const char* paged_decode_attention(const DecodeArgs& a, cudaStream_t s) {
  if (a.H % a.KV) return "paged_decode_attention: heads must be a multiple of kv heads";
  if (a.D == 128) return launch_decode<128>(a, s);
  if (a.D == 64) return launch_decode<64>(a, s);
  return "paged_decode_attention: head_dim must be 64 or 128";
}

}  // namespace nc

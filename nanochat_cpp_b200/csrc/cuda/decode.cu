// Inference kernels for the paged KV cache: append new keys / values into 16-token pages, and single-query
// attention over the pages (one query token per sequence, GQA, causal + left window).
//
// The reference decodes one row at a time over a contiguous cache and runs the attention through batched
// cuBLAS products (src/generate.cc:266-412, backends/cuda/kernels/attention_dispatch.h:38-48). Decode attention
// is bandwidth-bound (every cached key and value is read once per step), so this kernel streams K and V pages
// with 16-byte loads and keeps the online softmax in fp32 registers: CTAs cover (key split, kv head, sequence),
// the query heads of a group share the K / V traffic, and a small combine kernel merges the key splits.
#include "host_build.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "decode.h"

#include <atomic>

#ifndef NC_EMU
#include "pdl_launch.h"
#endif

namespace nc {

namespace {
std::atomic<bool> g_pdl{false};
}
bool pdl_enabled() { return g_pdl.load(std::memory_order_relaxed); }
void set_pdl_enabled(bool on) { g_pdl.store(on, std::memory_order_relaxed); }

namespace {
constexpr int kErrBadIndex = 7;   // status word: a position or page index outside its table (same code as ptx.cuh)

__global__ void __launch_bounds__(256) kv_append_kernel(__nv_bfloat16* __restrict__ k_pool,
                                                        __nv_bfloat16* __restrict__ v_pool,
                                                        const int* __restrict__ page_table, int max_pages,
                                                        const int* __restrict__ positions,
                                                        const __nv_bfloat16* __restrict__ k_new, long long k_ld,
                                                        const __nv_bfloat16* __restrict__ v_new, long long v_ld,
                                                        int tokens_per_seq, int total_tokens, int page_size,
                                                        int row_elems, int num_pages, int* status) {
  const int tok = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= total_tokens) return;
  const int lane = threadIdx.x & 31;
  const int pos = positions[tok];
  if (pos < 0) return;
  const int b = tok / tokens_per_seq;
  if (pos / page_size >= max_pages) {   // beyond the sequence's page table: nothing is written
    if (lane == 0 && status != nullptr) atomicCAS(status, 0, kErrBadIndex);
    return;
  }
  const int page = page_table[b * max_pages + pos / page_size];
  if (page < 0 || (num_pages > 0 && page >= num_pages)) {
    if (lane == 0 && status != nullptr) atomicCAS(status, 0, kErrBadIndex);
    return;
  }
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

constexpr int kDecodeWarps = 4;
constexpr int kDecodeUnroll = 4;

__device__ __forceinline__ void unpack8(const uint4& r, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 r;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return r;
}

// grid (splits, KV heads, B), 128 threads. A key row (D bf16) is read by D/8 lanes with one 16-byte load each, so a
// warp covers 32/(D/8) keys per load instruction and every thread keeps kDecodeUnroll K and V loads in flight. Each
// lane group runs its own online softmax over the keys it sees (fp32, base-2); the groups of the CTA are merged
// through shared memory at the end. With more than one split the CTA stores its unnormalised partial sums and the
// combine kernel finishes; with one split it writes the output row itself.
template <int D, int G>
__global__ void __launch_bounds__(kDecodeWarps * 32) paged_decode_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
    const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ page_table, int max_pages,
    const int* __restrict__ seq_lens, int H, int KV, int page_size, int window_left, float scale_log2, int splits,
    float* __restrict__ part_acc, float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
    long long q_stride_b) {
  constexpr int LPK = D / 8;        // lanes per key
  constexpr int KPW = 32 / LPK;     // keys per warp per load
  constexpr int GROUPS = kDecodeWarps * KPW;
  __shared__ float sm_m[G][GROUPS], sm_l[G][GROUPS];
  __shared__ float sm_acc[G][GROUPS][D];
  // the projection GEMM behind this kernel (programmatic serialization) may set itself up while keys are streamed
  NC_PDL_PROLOGUE();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  // a length beyond what the page table covers is clamped: the table is never indexed out of range
  const int len = min(seq_lens[b], max_pages * page_size);
  if (len <= 0) return;
  const int qpos = len - 1;
  const int first = window_left >= 0 ? max(0, qpos - window_left) : 0;
  const int n = qpos - first + 1;
  const int per = (n + splits - 1) / splits;
  const int k0 = first + split * per;
  const int k1 = min(k0 + per, qpos + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPK, part = lane % LPK;
  const int group = warp * KPW + sub;

  float qf[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint4 r = *reinterpret_cast<const uint4*>(q + b * q_stride_b + (kvh * G + g) * D + part * 8);
    unpack8(r, qf[g]);
#pragma unroll
    for (int i = 0; i < 8; ++i) qf[g][i] *= scale_log2;
  }
  float m[G], l[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -CUDART_INF_F, l[g] = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.0f;
  }
  const long long row = static_cast<long long>(KV) * D;
  const int* table = page_table + static_cast<long long>(b) * max_pages;
  // Software pipeline: the K and V rows of the next batch of keys (and the page-table entries their addresses need)
  // are requested before the current batch is reduced, so loads stay in flight during the arithmetic.
  auto fetch = [&](int kb, uint4 (&kr)[kDecodeUnroll], uint4 (&vr)[kDecodeUnroll], bool (&ok)[kDecodeUnroll]) {
#pragma unroll
    for (int u = 0; u < kDecodeUnroll; ++u) {
      const int key = kb + u * GROUPS + group;
      ok[u] = key < k1;
      kr[u] = make_uint4(0, 0, 0, 0), vr[u] = make_uint4(0, 0, 0, 0);
      if (ok[u]) {
        const int page = table[key / page_size];
        const long long off = (static_cast<long long>(page) * page_size + key % page_size) * row + kvh * D + part * 8;
        kr[u] = *reinterpret_cast<const uint4*>(k_pool + off);
        vr[u] = *reinterpret_cast<const uint4*>(v_pool + off);
      }
    }
  };
  uint4 kr[kDecodeUnroll], vr[kDecodeUnroll];
  bool ok[kDecodeUnroll];
  fetch(k0, kr, vr, ok);
  for (int kb = k0; kb < k1; kb += GROUPS * kDecodeUnroll) {  // uniform over the CTA: the shuffles below are full-warp
    uint4 kr_next[kDecodeUnroll], vr_next[kDecodeUnroll];
    bool ok_next[kDecodeUnroll];
    fetch(kb + GROUPS * kDecodeUnroll, kr_next, vr_next, ok_next);   // past k1 every key is masked: no load is issued
    float sc[kDecodeUnroll][G];
#pragma unroll
    for (int u = 0; u < kDecodeUnroll; ++u) {
      float kf[8];
      unpack8(kr[u], kf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) d = fmaf(qf[g][i], kf[i], d);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        sc[u][g] = ok[u] ? d : -CUDART_INF_F;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = m[g];
#pragma unroll
      for (int u = 0; u < kDecodeUnroll; ++u) mx = fmaxf(mx, sc[u][g]);
      if (mx == -CUDART_INF_F) continue;
      const float alpha = exp2f(m[g] - mx);  // 0 when m is still -inf
      l[g] *= alpha;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[g][i] *= alpha;
      m[g] = mx;
    }
#pragma unroll
    for (int u = 0; u < kDecodeUnroll; ++u) {
      float vf[8];
      unpack8(vr[u], vf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float p = sc[u][g] == -CUDART_INF_F ? 0.0f : exp2f(sc[u][g] - m[g]);
        l[g] += p;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(p, vf[i], acc[g][i]);
      }
    }
#pragma unroll
    for (int u = 0; u < kDecodeUnroll; ++u) kr[u] = kr_next[u], vr[u] = vr_next[u], ok[u] = ok_next[u];
  }
  // merge the lane groups
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (part == 0) sm_m[g][group] = m[g], sm_l[g][group] = l[g];
#pragma unroll
    for (int i = 0; i < 8; ++i) sm_acc[g][group][part * 8 + i] = acc[g][i];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += kDecodeWarps * 32) {
    const int g = idx / D, d = idx % D;
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < GROUPS; ++j) mx = fmaxf(mx, sm_m[g][j]);
    float a = 0.0f, ls = 0.0f;
    if (mx != -CUDART_INF_F) {
#pragma unroll
      for (int j = 0; j < GROUPS; ++j) {
        const float w = exp2f(sm_m[g][j] - mx);
        a = fmaf(w, sm_acc[g][j][d], a);
        ls = fmaf(w, sm_l[g][j], ls);
      }
    }
    const long long head = static_cast<long long>(b) * H + kvh * G + g;
    if (splits == 1) {
      out[head * D + d] = __float2bfloat16_rn(ls > 0.0f ? a / ls : 0.0f);
    } else {
      part_acc[(head * splits + split) * D + d] = a;
      if (d == 0) {
        part_ml[(head * splits + split) * 2] = mx;
        part_ml[(head * splits + split) * 2 + 1] = ls;
      }
    }
  }
}

// grid (H, B), D threads: out = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
template <int D>
__global__ void __launch_bounds__(D) decode_combine_kernel(const float* __restrict__ part_acc,
                                                           const float* __restrict__ part_ml,
                                                           const int* __restrict__ seq_lens, int H, int splits,
                                                           __nv_bfloat16* __restrict__ out) {
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  if (seq_lens[b] <= 0) return;
  const long long head = static_cast<long long>(b) * H + h;
  float mx = -CUDART_INF_F;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part_ml[(head * splits + s) * 2]);
  float a = 0.0f, ls = 0.0f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(head * splits + s) * 2];
    if (ms == -CUDART_INF_F) continue;
    const float w = exp2f(ms - mx);
    a = fmaf(w, part_acc[(head * splits + s) * D + d], a);
    ls = fmaf(w, part_ml[(head * splits + s) * 2 + 1], ls);
  }
  out[head * D + d] = __float2bfloat16_rn(ls > 0.0f ? a / ls : 0.0f);
}

#ifndef NC_EMU
template <int D>
const char* launch_decode(const DecodeArgs& a, cudaStream_t s) {
  const int splits = a.splits < 1 ? 1 : a.splits;
  if (splits > 1 && (a.part_acc == nullptr || a.part_ml == nullptr)) return "paged_decode_attention: no split scratch";
  const dim3 grid(splits, a.KV, a.B);
  const int G = a.H / a.KV;
  const float sl2 = a.scale * 1.4426950408889634f;
#define NC_DECODE(GV)                                                                                                \
  launch_maybe_pdl(paged_decode_kernel<D, GV>, grid, dim3(kDecodeWarps * 32), 0, s, a.q, a.k_pool, a.v_pool,          \
                   a.page_table, a.max_pages, a.seq_lens, a.H, a.KV, a.page_size, a.window_left, sl2, splits,        \
                   a.part_acc, a.part_ml, a.out, a.q_stride_b > 0 ? a.q_stride_b : static_cast<long long>(a.H) * D)
  switch (G) {
    case 1: NC_DECODE(1); break;
    case 2: NC_DECODE(2); break;
    case 4: NC_DECODE(4); break;
    case 8: NC_DECODE(8); break;
    default: return "paged_decode_attention: group size must be 1, 2, 4 or 8";
  }
#undef NC_DECODE
  if (splits > 1)
    decode_combine_kernel<D><<<dim3(a.H, a.B), D, 0, s>>>(a.part_acc, a.part_ml, a.seq_lens, a.H, splits, a.out);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}
#endif  // !NC_EMU

}  // namespace

// Decode prologue in one launch (head_dim 128, one new token per sequence): for the token's fused QKV row,
// q and k heads get head RMSNorm -> RoPE at the token's position -> scale (the arithmetic of the training kernel
// qk_prep_fwd, rounding points included); q goes to a dense [B, H, D] buffer, k straight into its page of the
// cache, and the value row (which may come from another buffer: the value gate writes its own) is copied into its
// page as well. One warp per (token, four heads) plus one warp per token for the value row; eight lanes share a head.
__global__ void __launch_bounds__(256) decode_prep_append_kernel(
    const __nv_bfloat16* __restrict__ qk, long long ld_qk, const __nv_bfloat16* __restrict__ v, long long ld_v,
    const float* __restrict__ cosT, const float* __restrict__ sinT, const int* __restrict__ positions,
    const int* __restrict__ page_table, int max_pages, int page_size, __nv_bfloat16* __restrict__ q_out,
    __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, int tokens, int H, int KV, float eps,
    float scale, int num_pages, int* status) {
  constexpr int D = 128;
  NC_PDL_PROLOGUE();
  const int groups = (H + KV + 3) / 4;                  // head groups of the q / k part
  const int unit = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (unit >= tokens * (groups + 1)) return;
  const int tok = unit / (groups + 1), grp = unit % (groups + 1);
  const int lane = threadIdx.x & 31;
  const int pos = positions[tok];
  if (pos < 0) return;
  const bool page_ok = pos / page_size < max_pages;
  const int page = page_ok ? page_table[static_cast<long long>(tok) * max_pages + pos / page_size] : -1;
  // a position past the page table or a page outside the pool: q is still produced, nothing goes to the cache
  const bool cache_ok = page >= 0 && (num_pages <= 0 || page < num_pages);
  if (!cache_ok && lane == 0 && status != nullptr) atomicCAS(status, 0, kErrBadIndex);
  const long long cache_row = (static_cast<long long>(page) * page_size + pos % page_size) * KV * D;
  if (grp == groups) {   // value row -> cache
    if (!cache_ok) return;
    const uint4* src = reinterpret_cast<const uint4*>(v + static_cast<long long>(tok) * ld_v);
    uint4* dst = reinterpret_cast<uint4*>(v_pool + cache_row);
    for (int i = lane; i < KV * D / 8; i += 32) dst[i] = src[i];
    return;
  }
  const int sub = lane >> 3, j = lane & 7;
  const int h = grp * 4 + sub;
  const bool act = h < H + KV;
  const float* cp = cosT + static_cast<long long>(pos) * (D / 2);
  const float* sp = sinT + static_cast<long long>(pos) * (D / 2);
  float c[8], sn[8];
  *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cp + 8 * j);
  *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cp + 8 * j + 4);
  *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sp + 8 * j);
  *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sp + 8 * j + 4);
  const __nv_bfloat16* row_in = qk + static_cast<long long>(tok) * ld_qk;
  float a[8], b[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) a[e] = 0.f, b[e] = 0.f;
  if (act) {
    unpack8(*reinterpret_cast<const uint4*>(row_in + h * D + 8 * j), a);
    unpack8(*reinterpret_cast<const uint4*>(row_in + h * D + 64 + 8 * j), b);
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss += a[e] * a[e] + b[e] * b[e];
  ss += __shfl_xor_sync(0xffffffffu, ss, 4);
  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
  const float r = 1.0f / sqrtf(ss * (1.0f / static_cast<float>(D)) + eps);
  if (!act) return;
  float y1[8], y2[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float x1 = __bfloat162float(__float2bfloat16_rn(a[e] * r)), x2 = __bfloat162float(__float2bfloat16_rn(b[e] * r));
    y1[e] = (x1 * c[e] + x2 * sn[e]) * scale;
    y2[e] = (-x1 * sn[e] + x2 * c[e]) * scale;
  }
  if (h >= H && !cache_ok) return;
  __nv_bfloat16* dst = h < H ? q_out + (static_cast<long long>(tok) * H + h) * D : k_pool + cache_row + (h - H) * D;
  *reinterpret_cast<uint4*>(dst + 8 * j) = pack8(y1);
  *reinterpret_cast<uint4*>(dst + 64 + 8 * j) = pack8(y2);
}

#ifndef NC_EMU
void kv_append(__nv_bfloat16* k_pool, __nv_bfloat16* v_pool, const int* page_table, int max_pages,
               const int* positions, const __nv_bfloat16* k_new, long long k_ld, const __nv_bfloat16* v_new,
               long long v_ld, int B, int T, int page_size, int row_elems, cudaStream_t s, int num_pages, int* status) {
  const int total = B * T;
  if (total <= 0) return;
  kv_append_kernel<<<(total + 7) / 8, 256, 0, s>>>(k_pool, v_pool, page_table, max_pages, positions, k_new, k_ld,
                                                   v_new, v_ld, T, total, page_size, row_elems, num_pages, status);
}
#endif  // !NC_EMU

// fp32 out[r, c] = cap * tanh(logits[r, c] / cap) for c < vocab: the head's soft cap, one pass over the bf16 logits
// (two elements per thread; the same float operations as the elementwise definition).
__global__ void __launch_bounds__(256) softcap_logits_kernel(const __nv_bfloat16* __restrict__ lg, long long ld,
                                                             float* __restrict__ out, int rows, int vocab, float cap) {
  const long long i = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) * 2;
  const int r = static_cast<int>(i / vocab), c = static_cast<int>(i % vocab);
  if (r >= rows) return;
  const __nv_bfloat16* src = lg + static_cast<long long>(r) * ld + c;
  float* dst = out + static_cast<long long>(r) * vocab + c;
  dst[0] = cap * tanhf(__bfloat162float(src[0]) / cap);
  if (c + 1 < vocab) dst[1] = cap * tanhf(__bfloat162float(src[1]) / cap);
}
#ifndef NC_EMU
void softcap_logits(const __nv_bfloat16* lg, long long ld, float* out, int rows, int vocab, float cap, cudaStream_t s) {
  if (rows <= 0 || vocab <= 0) return;
  const long long pairs = (static_cast<long long>(rows) * vocab + 1) / 2;   // vocab even: pairs never straddle rows
  softcap_logits_kernel<<<static_cast<unsigned>((pairs + 255) / 256), 256, 0, s>>>(lg, ld, out, rows, vocab, cap);
}

#endif  // !NC_EMU
// out[r] = index of the largest of logits[r, 0 .. vocab): greedy decoding straight from the bf16 logits (the soft
// cap is monotonic, so the fp32 capped copy is not needed). Ties go to the lowest index, as in the definition.
__global__ void __launch_bounds__(256) argmax_rows_kernel(const __nv_bfloat16* __restrict__ lg, long long ld, int vocab,
                                                          long long* __restrict__ out) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const __nv_bfloat16* row = lg + static_cast<long long>(blockIdx.x) * ld;
  float best = -CUDART_INF_F;
  int arg = 0x7fffffff;
  const bool vec = (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(lg) & 15) == 0);
  const int vend = vec ? (vocab / 8) * 8 : 0;
  for (int c = threadIdx.x * 8; c < vend; c += 256 * 8) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(row + c), f);
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (f[e] > best) best = f[e], arg = c + e;   // ascending scan: the first of equal values stays
  }
  for (int c = vend + threadIdx.x; c < vocab; c += 256) {
    const float v = __bfloat162float(row[c]);
    if (v > best || (v == best && c < arg)) best = v, arg = c;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
    if (ov > best || (ov == best && oi < arg)) best = ov, arg = oi;
  }
  if ((threadIdx.x & 31) == 0) sv[threadIdx.x >> 5] = best, si[threadIdx.x >> 5] = arg;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < arg)) best = sv[w], arg = si[w];
    out[blockIdx.x] = arg == 0x7fffffff ? 0 : arg;   // a row of NaNs or -inf: index 0
  }
}
#ifndef NC_EMU
void argmax_rows(const __nv_bfloat16* lg, long long ld, long long* out, int rows, int vocab, cudaStream_t s) {
  if (rows <= 0 || vocab <= 0) return;
  argmax_rows_kernel<<<rows, 256, 0, s>>>(lg, ld, vocab, out);
}
#endif  // !NC_EMU

#ifndef NC_EMU
const char* decode_prep_append(const __nv_bfloat16* qk, long long ld_qk, const __nv_bfloat16* v, long long ld_v,
                               const float* cosT, const float* sinT, const int* positions, const int* page_table,
                               int max_pages, int page_size, __nv_bfloat16* q_out, __nv_bfloat16* k_pool,
                               __nv_bfloat16* v_pool, int tokens, int H, int KV, int D, float eps, float scale,
                               cudaStream_t s, int num_pages, int* status) {
  if (tokens <= 0) return nullptr;
  if (D != 128) return "decode_prep_append: head_dim must be 128";
  if (ld_qk % 8 || ld_v % 8 ||
      ((reinterpret_cast<uintptr_t>(qk) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(q_out) |
        reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool) | reinterpret_cast<uintptr_t>(cosT) |
        reinterpret_cast<uintptr_t>(sinT)) & 15))
    return "decode_prep_append: rows must be 16-byte aligned";
  const int units = tokens * ((H + KV + 3) / 4 + 1);
  const cudaError_t e = launch_maybe_pdl(decode_prep_append_kernel, dim3((units + 7) / 8), dim3(256), 0, s, qk, ld_qk, v,
                                         ld_v, cosT, sinT, positions, page_table, max_pages, page_size, q_out, k_pool,
                                         v_pool, tokens, H, KV, eps, scale, num_pages, status);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}
#endif  // !NC_EMU

int decode_splits(int B, int KV, int max_keys) {
  const int target = 148 * 4;  // four 128-thread CTAs per SM keep enough loads in flight
  int splits = (target + B * KV - 1) / (B * KV);
  const int by_len = (max_keys + 255) / 256;  // at least 256 keys per split
  if (splits > by_len) splits = by_len;
  if (splits > 32) splits = 32;
  return splits < 1 ? 1 : splits;
}

#ifndef NC_EMU
const char* paged_decode_attention(const DecodeArgs& a, cudaStream_t s) {
  if (a.H % a.KV) return "paged_decode_attention: heads must be a multiple of kv heads";
  if (a.D == 128) return launch_decode<128>(a, s);
  if (a.D == 64) return launch_decode<64>(a, s);
  return "paged_decode_attention: head_dim must be 64 or 128";
}
#endif  // !NC_EMU

}  // namespace nc

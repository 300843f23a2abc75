// Memory-bound row kernels: norms, residual blends, QK preparation, value gate, smear, embeddings,
// softcap + cross entropy, gradient-norm reduction. One warp owns one row (or one head of one token) and
// moves 16-byte vectors; statistics are reduced with shuffles in fp32. These replace the reference's
// one-block-per-row kernels and its pointwise composition tier (reference backends/cuda/kernels/
// rms_norm.cu, qk_prep.cu, pointwise.cu, value_gate.cu, smear.cu, embedding.cu, classifier.cu,
// grad_norm.cu) with fewer, wider passes: e.g. the residual blend and the pre-attention norm are one
// kernel, and the classifier forward and backward are one sweep over a logits chunk.
#include "host_build.h"

#include "rowops.h"

#include "mx_quant.cuh"
#ifndef NC_EMU
#include "pdl_launch.h"
#endif

#include <math_constants.h>

namespace nc {

namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = kWarpsPerBlock * 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

struct V8 {
  float f[8];
};
__device__ __forceinline__ V8 ld8(const bf16* p) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
  V8 v;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v.f[2 * i] = __uint_as_float(w[i] << 16);
    v.f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
  return v;
}
__device__ __forceinline__ void st8(bf16* p, const V8& v) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 t = __floats2bfloat162_rn(v.f[2 * i], v.f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&t);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ float b2f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 f2b(float v) { return __float2bfloat16_rn(v); }
__host__ __device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? sh[threadIdx.x] : 0.0f;
  if (warp == 0) t = warp_sum(t);
  if (threadIdx.x == 0) sh[0] = t;
  __syncthreads();
  t = sh[0];
  __syncthreads();
  return t;
}

inline int blocks_for_rows(long long rows) { return static_cast<int>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock); }

// ------------------------------------------------------------------ RMSNorm family
// MODE 0: y = norm(x), save rstd.  MODE 1: y = x*rstd (recompute).  MODE 2: blend: xr = a*x + b*x0, h = norm(xr).
template <int MODE>
__global__ void __launch_bounds__(kThreads) rmsnorm_kernel(const bf16* __restrict__ x, long long ldx,
                                                           const bf16* __restrict__ x0, const float* lam_r,
                                                           const float* lam_0, bf16* __restrict__ xr,
                                                           bf16* __restrict__ y, float* __restrict__ rstd, int rows,
                                                           int dim, float eps, uint8_t* __restrict__ yq = nullptr,
                                                           uint8_t* __restrict__ sf = nullptr) {
  // a GEMM launched behind this kernel with programmatic serialization may set itself up while the rows are normed
  NC_PDL_PROLOGUE();
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const bf16* xp = x + static_cast<long long>(row) * ldx;
  bf16* yp = y + static_cast<long long>(row) * dim;
  const bool vec = (dim % 8 == 0) && aligned16(xp) && aligned16(yp) && (ldx % 8 == 0);
  float a = 1.0f, b = 0.0f;
  const bf16* x0p = nullptr;
  bf16* xrp = nullptr;
  if (MODE == 2) {
    a = *lam_r;
    b = *lam_0;
    x0p = x0 + static_cast<long long>(row) * dim;
    xrp = xr + static_cast<long long>(row) * dim;
  }
  float r;
  if (MODE == 1) {
    r = rstd[row];
  } else {
    float ss = 0.0f;
    if (vec) {
      for (int i = lane * 8; i < dim; i += 256) {
        V8 v = ld8(xp + i);
        if (MODE == 2) {
          const V8 w = ld8(x0p + i);
#pragma unroll
          for (int e = 0; e < 8; ++e) v.f[e] = b2f(f2b(a * v.f[e] + b * w.f[e]));
          st8(xrp + i, v);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += v.f[e] * v.f[e];
      }
    } else {
      for (int i = lane; i < dim; i += 32) {
        float v = b2f(xp[i]);
        if (MODE == 2) {
          v = b2f(f2b(a * v + b * b2f(x0p[i])));
          xrp[i] = f2b(v);
        }
        ss += v * v;
      }
    }
    ss = warp_sum(ss);
    r = 1.0f / sqrtf(ss * (1.0f / static_cast<float>(dim)) + eps);
    if (lane == 0) rstd[row] = r;
  }
  if (MODE == 2) __syncwarp();
  const bf16* src = (MODE == 2) ? xrp : xp;
  if (yq != nullptr) {
    // MXFP8 copy of the output beside the bf16 one (host guarantees the vector path and dim % 128 == 0): the four
    // lanes of a 32-element block agree on its power-of-two scale, the bf16-rounded values are encoded as E4M3, and
    // the scale bytes go straight into the 512-byte atoms the GEMM copies into tensor memory (128-row groups).
    // The trip count is the same for every lane, so the shuffles stay warp-uniform when dim % 256 == 128.
    const int kbs = dim >> 7;
    for (int base = 0; base < dim; base += 256) {
      const int i = base + lane * 8;
      const bool act = i < dim;
      float f[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
      float amax = 0.0f;
      if (act) {
        V8 v = ld8(src + i);
#pragma unroll
        for (int e = 0; e < 8; ++e) v.f[e] *= r;
        st8(yp + i, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          f[e] = b2f(f2b(v.f[e]));
          amax = fmaxf(amax, fabsf(f[e]));
        }
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const uint32_t eb = mx_block_exponent(amax);
      if (act) *reinterpret_cast<uint2*>(yq + static_cast<long long>(row) * dim + i) = mx_pack8(f, mx_inverse_scale(eb));
      const int first = lane & 16;
      const uint32_t b0 = __shfl_sync(0xffffffffu, eb, first), b1 = __shfl_sync(0xffffffffu, eb, first + 4);
      const uint32_t b2 = __shfl_sync(0xffffffffu, eb, first + 8), b3 = __shfl_sync(0xffffffffu, eb, first + 12);
      if (act && (lane & 15) == 0) {
        const long long atom = static_cast<long long>(row >> 7) * kbs + (i >> 7);
        *reinterpret_cast<uint32_t*>(sf + atom * 512 + mx_atom_offset(row & 127)) = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
      }
    }
  } else if (vec) {
    for (int i = lane * 8; i < dim; i += 256) {
      V8 v = ld8(src + i);
#pragma unroll
      for (int e = 0; e < 8; ++e) v.f[e] *= r;
      st8(yp + i, v);
    }
  } else {
    for (int i = lane; i < dim; i += 32) yp[i] = f2b(b2f(src[i]) * r);
  }
}

__global__ void __launch_bounds__(kThreads) rmsnorm_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy,
                                                               const float* __restrict__ rstd,
                                                               const bf16* __restrict__ residual,
                                                               bf16* __restrict__ dx, int rows, int dim) {
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long off = static_cast<long long>(row) * dim;
  const bf16 *xp = x + off, *dyp = dy + off;
  const bf16* rp = residual ? residual + off : nullptr;
  bf16* dxp = dx + off;
  const bool vec = (dim % 8 == 0) && aligned16(xp) && aligned16(dyp) && aligned16(dxp) && (!rp || aligned16(rp));
  float dot = 0.0f;
  if (vec) {
    for (int i = lane * 8; i < dim; i += 256) {
      const V8 a = ld8(xp + i), g = ld8(dyp + i);
#pragma unroll
      for (int e = 0; e < 8; ++e) dot += a.f[e] * g.f[e];
    }
  } else {
    for (int i = lane; i < dim; i += 32) dot += b2f(xp[i]) * b2f(dyp[i]);
  }
  dot = warp_sum(dot);
  const float r = rstd[row];
  const float coeff = r * r * r * dot * (1.0f / static_cast<float>(dim));
  if (vec) {
    for (int i = lane * 8; i < dim; i += 256) {
      const V8 a = ld8(xp + i), g = ld8(dyp + i);
      V8 o;
#pragma unroll
      for (int e = 0; e < 8; ++e) o.f[e] = r * g.f[e] - coeff * a.f[e];
      if (rp) {
        const V8 q = ld8(rp + i);
#pragma unroll
        for (int e = 0; e < 8; ++e) o.f[e] += q.f[e];
      }
      st8(dxp + i, o);
    }
  } else {
    for (int i = lane; i < dim; i += 32) {
      float o = r * b2f(dyp[i]) - coeff * b2f(xp[i]);
      if (rp) o += b2f(rp[i]);
      dxp[i] = f2b(o);
    }
  }
}

// Backward of h = rmsnorm(xr), xr = lam_r * x + lam_0 * x0, in one pass over the row:
//   dxr = rstd * dh' - rstd^3 <xr, dh'> / dim * xr + residual      (dh' = dh with `extra` added to its first columns)
//   dx = lam_r * dxr;  dx0 (+)= lam_0 * dxr;  g_lam_r += <dxr, x>;  g_lam_0 += <dxr, x0>
// dxr never reaches memory (the unfused pair writes it as bf16 and reads it back), the scalar gradients go straight
// into the flat gradient buffer, and the separate pass that added the value-gate's 12 columns into dh is folded in.
__global__ void __launch_bounds__(kThreads) norm_blend_bwd_kernel(
    const bf16* __restrict__ xr, const bf16* __restrict__ dh, const float* __restrict__ rstd,
    const bf16* __restrict__ residual, const float* __restrict__ extra, int extra_cols, const bf16* __restrict__ x,
    const bf16* __restrict__ x0, const float* __restrict__ lam_r, const float* __restrict__ lam_0,
    bf16* __restrict__ dx, bf16* __restrict__ dx0, int accumulate_dx0, float* __restrict__ g_lam_r,
    float* __restrict__ g_lam_0, int rows, int dim) {
  __shared__ float sh[2][kWarpsPerBlock];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerBlock + warp;
  float acc_r = 0.0f, acc_0 = 0.0f;
  if (row < rows) {
    const long long off = static_cast<long long>(row) * dim;
    const float* ex = extra != nullptr ? extra + static_cast<long long>(row) * extra_cols : nullptr;
    auto load_dh = [&](int i) {
      V8 g = ld8(dh + off + i);
      if (ex != nullptr && i < extra_cols) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (i + e < extra_cols) g.f[e] = b2f(f2b(g.f[e] + ex[i + e]));   // the unfused path rounds this sum to bf16
      }
      return g;
    };
    float dot = 0.0f;
    for (int i = lane * 8; i < dim; i += 256) {
      const V8 a = ld8(xr + off + i), g = load_dh(i);
#pragma unroll
      for (int e = 0; e < 8; ++e) dot += a.f[e] * g.f[e];
    }
    dot = warp_sum(dot);
    const float r = rstd[row];
    const float coeff = r * r * r * dot * (1.0f / static_cast<float>(dim));
    const float kr = *lam_r, k0 = *lam_0;
    for (int i = lane * 8; i < dim; i += 256) {
      const V8 a = ld8(xr + off + i), g = load_dh(i), q = ld8(residual + off + i);
      const V8 xv = ld8(x + off + i), x0v = ld8(x0 + off + i);
      V8 d, d0;
      if (accumulate_dx0) d0 = ld8(dx0 + off + i);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float t = r * g.f[e] - coeff * a.f[e] + q.f[e];
        acc_r += t * xv.f[e];
        acc_0 += t * x0v.f[e];
        d.f[e] = kr * t;
        d0.f[e] = (accumulate_dx0 ? d0.f[e] : 0.0f) + k0 * t;
      }
      st8(dx + off + i, d);
      st8(dx0 + off + i, d0);
    }
  }
  acc_r = warp_sum(acc_r);
  acc_0 = warp_sum(acc_0);
  if (lane == 0) sh[0][warp] = acc_r, sh[1][warp] = acc_0;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.0f, b = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarpsPerBlock; ++w) a += sh[0][w], b += sh[1][w];
    atomicAdd(g_lam_r, a);
    atomicAdd(g_lam_0, b);
  }
}

// ------------------------------------------------------------------ flat elementwise + dot reductions
// KIND 0: blend_bwd   KIND 1: backout_fwd   KIND 2: backout_bwd   KIND 3: add
template <int KIND>
__global__ void __launch_bounds__(256) flat_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b,
                                                   const bf16* __restrict__ c, const float* s0, const float* s1,
                                                   bf16* __restrict__ o0, bf16* __restrict__ o1, int flag,
                                                   float* red, long long n) {
  __shared__ float sh[32];
  const float k0 = s0 ? *s0 : 0.0f;
  const float k1 = s1 ? *s1 : 0.0f;
  float acc0 = 0.0f, acc1 = 0.0f;
  const long long nv = n / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e0 = i * 8;
    if (KIND == 0) {  // a=dxr, b=x, c=x0; o0=dx, o1=dx0 (accumulate if flag)
      const V8 g = ld8(a + e0), xv = ld8(b + e0), x0v = ld8(c + e0);
      V8 d, d0;
      if (flag) d0 = ld8(o1 + e0);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        acc0 += g.f[e] * xv.f[e];
        acc1 += g.f[e] * x0v.f[e];
        d.f[e] = k0 * g.f[e];
        d0.f[e] = (flag ? d0.f[e] : 0.0f) + k1 * g.f[e];
      }
      st8(o0 + e0, d);
      st8(o1 + e0, d0);
    } else if (KIND == 1) {  // y = a - k0*b
      const V8 xv = ld8(a + e0), bv = ld8(b + e0);
      V8 y;
#pragma unroll
      for (int e = 0; e < 8; ++e) y.f[e] = xv.f[e] - k0 * bv.f[e];
      st8(o0 + e0, y);
    } else if (KIND == 2) {  // a=dy, b=xb: o0 = -k0*dy ; red -= <dy,xb>
      const V8 g = ld8(a + e0), bv = ld8(b + e0);
      V8 y;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        acc0 -= g.f[e] * bv.f[e];
        y.f[e] = -k0 * g.f[e];
      }
      st8(o0 + e0, y);
    } else {
      const V8 xv = ld8(a + e0), bv = ld8(b + e0);
      V8 y;
#pragma unroll
      for (int e = 0; e < 8; ++e) y.f[e] = xv.f[e] + bv.f[e];
      st8(o0 + e0, y);
    }
  }
  // scalar tail
  if (blockIdx.x == 0) {
    for (long long e0 = nv * 8 + threadIdx.x; e0 < n; e0 += blockDim.x) {
      if (KIND == 0) {
        const float g = b2f(a[e0]);
        acc0 += g * b2f(b[e0]);
        acc1 += g * b2f(c[e0]);
        o0[e0] = f2b(k0 * g);
        o1[e0] = f2b((flag ? b2f(o1[e0]) : 0.0f) + k1 * g);
      } else if (KIND == 1) {
        o0[e0] = f2b(b2f(a[e0]) - k0 * b2f(b[e0]));
      } else if (KIND == 2) {
        acc0 -= b2f(a[e0]) * b2f(b[e0]);
        o0[e0] = f2b(-k0 * b2f(a[e0]));
      } else {
        o0[e0] = f2b(b2f(a[e0]) + b2f(b[e0]));
      }
    }
  }
  if (KIND == 0 || KIND == 2) {
    acc0 = block_sum(acc0, sh);
    if (KIND == 0) acc1 = block_sum(acc1, sh);
    if (threadIdx.x == 0) {
      atomicAdd(red, acc0);
      if (KIND == 0) atomicAdd(red + 1, acc1);
    }
  }
}

__global__ void add_cols_kernel(bf16* dh, long long ld, const float* extra, int rows, int ncols) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * ncols) return;
  const int r = i / ncols, c = i % ncols;
  bf16* p = dh + static_cast<long long>(r) * ld + c;
  *p = f2b(b2f(*p) + extra[i]);
}

// ------------------------------------------------------------------ QK preparation
// One warp per token walks every head of the row, so the rotary row (cos/sin of the token's position)
// is loaded once and reused by all heads. Forward: y = rope(norm(x)) * scale.
// Both kernels are bound by memory latency, so resident warps count for more than registers: the launch bounds ask
// for six (forward) and four (backward) blocks per SM, which took them from 0.81 / 0.75 to 0.87 / 0.82 of the measured
// copy rate; one block more on the backward side spills enough to lose it again (0.67).
__global__ void __launch_bounds__(kThreads, 6) qk_prep_fwd_kernel(const bf16* __restrict__ in, long long ld_in,
                                                               bf16* __restrict__ out, long long ld_out,
                                                               const float* __restrict__ cosT,
                                                               const float* __restrict__ sinT, const int* positions,
                                                               int tokens, int seq, int heads, int D, float eps,
                                                               float scale) {
  const int tok = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (tok >= tokens) return;
  const int lane = threadIdx.x & 31;
  const int pos = positions ? positions[tok] : tok % seq;
  const int half = D / 2;
  const bf16* row_in = in + static_cast<long long>(tok) * ld_in;
  bf16* row_out = out + static_cast<long long>(tok) * ld_out;
  const float* cp = cosT + static_cast<long long>(pos) * half;
  const float* sp = sinT + static_cast<long long>(pos) * half;
  const float inv_d = 1.0f / static_cast<float>(D);
  // head_dim 128: eight lanes share a head (16-byte loads of both halves), four heads per warp at a time
  if (D == 128 && ((reinterpret_cast<uintptr_t>(row_in) | reinterpret_cast<uintptr_t>(row_out)) & 15) == 0 &&
      ((reinterpret_cast<uintptr_t>(cp) | reinterpret_cast<uintptr_t>(sp)) & 15) == 0) {
    const int sub = lane >> 3, j = lane & 7;
    float c[8], sn[8];
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cp + 8 * j);
    *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cp + 8 * j + 4);
    *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sp + 8 * j);
    *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sp + 8 * j + 4);
#pragma unroll 2
    for (int h0 = 0; h0 < heads; h0 += 4) {
      const int h = h0 + sub;
      const bool act = h < heads;
      V8 a, b;
#pragma unroll
      for (int e = 0; e < 8; ++e) a.f[e] = 0.f, b.f[e] = 0.f;
      if (act) {
        a = ld8(row_in + h * 128 + 8 * j);
        b = ld8(row_in + h * 128 + 64 + 8 * j);
      }
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += a.f[e] * a.f[e] + b.f[e] * b.f[e];
      ss += __shfl_xor_sync(0xffffffffu, ss, 4);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      const float r = 1.0f / sqrtf(ss * inv_d + eps);
      if (act) {
        V8 y1, y2;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float x1 = b2f(f2b(a.f[e] * r)), x2 = b2f(f2b(b.f[e] * r));
          y1.f[e] = (x1 * c[e] + x2 * sn[e]) * scale;
          y2.f[e] = (-x1 * sn[e] + x2 * c[e]) * scale;
        }
        st8(row_out + h * 128 + 8 * j, y1);
        st8(row_out + h * 128 + 64 + 8 * j, y2);
      }
    }
    return;
  }
  const bool vec = (half % 2 == 0) && half <= 64 && (reinterpret_cast<uintptr_t>(cp) & 7) == 0 &&
                   (reinterpret_cast<uintptr_t>(sp) & 7) == 0 &&
                   ((reinterpret_cast<uintptr_t>(row_in) | reinterpret_cast<uintptr_t>(row_out)) & 3) == 0 && (D % 2 == 0);
  if (vec) {
    const int d = lane * 2;
    const bool act = d < half;
    float2 c = make_float2(0.f, 0.f), sn = make_float2(0.f, 0.f);
    if (act) {
      c = *reinterpret_cast<const float2*>(cp + d);
      sn = *reinterpret_cast<const float2*>(sp + d);
    }
    for (int h = 0; h < heads; ++h) {
      const bf16* xp = row_in + h * D;
      bf16* yp = row_out + h * D;
      float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
      if (act) {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(xp + d);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(xp + d + half);
        a0 = b2f(a.x), a1 = b2f(a.y), b0 = b2f(b.x), b1 = b2f(b.y);
      }
      const float ss = warp_sum(a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1);
      const float r = 1.0f / sqrtf(ss * inv_d + eps);
      if (act) {
        // the normalised value is rounded to bf16 before the rotation, as a separate norm pass would
        const float x10 = b2f(f2b(a0 * r)), x11 = b2f(f2b(a1 * r));
        const float x20 = b2f(f2b(b0 * r)), x21 = b2f(f2b(b1 * r));
        *reinterpret_cast<__nv_bfloat162*>(yp + d) =
            __floats2bfloat162_rn((x10 * c.x + x20 * sn.x) * scale, (x11 * c.y + x21 * sn.y) * scale);
        *reinterpret_cast<__nv_bfloat162*>(yp + d + half) =
            __floats2bfloat162_rn((-x10 * sn.x + x20 * c.x) * scale, (-x11 * sn.y + x21 * c.y) * scale);
      }
    }
    return;
  }
  for (int h = 0; h < heads; ++h) {
    const bf16* xp = row_in + h * D;
    bf16* yp = row_out + h * D;
    float ss = 0.0f;
    for (int d = lane; d < D; d += 32) {
      const float v = b2f(xp[d]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss * inv_d + eps);
    for (int d = lane; d < half; d += 32) {
      const float x1 = b2f(f2b(b2f(xp[d]) * r));
      const float x2 = b2f(f2b(b2f(xp[d + half]) * r));
      const float c = cp[d], s = sp[d];
      yp[d] = f2b((x1 * c + x2 * s) * scale);
      yp[d + half] = f2b((-x1 * s + x2 * c) * scale);
    }
  }
}

__global__ void __launch_bounds__(kThreads, 4) qk_prep_bwd_kernel(const bf16* __restrict__ pre, long long ld_pre,
                                                               const bf16* __restrict__ grad, long long ld_grad,
                                                               bf16* __restrict__ out, long long ld_out,
                                                               const float* __restrict__ cosT,
                                                               const float* __restrict__ sinT, int tokens, int seq,
                                                               int heads, int D, float eps, float scale) {
  const int tok = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (tok >= tokens) return;
  const int lane = threadIdx.x & 31;
  const int pos = tok % seq;
  const int half = D / 2;
  const bf16* row_x = pre + static_cast<long long>(tok) * ld_pre;
  const bf16* row_g = grad + static_cast<long long>(tok) * ld_grad;
  bf16* row_o = out + static_cast<long long>(tok) * ld_out;
  const float* cp = cosT + static_cast<long long>(pos) * half;
  const float* sp = sinT + static_cast<long long>(pos) * half;
  const float inv_d = 1.0f / static_cast<float>(D);
  if (D == 128 && ((reinterpret_cast<uintptr_t>(row_x) | reinterpret_cast<uintptr_t>(row_g) |
                    reinterpret_cast<uintptr_t>(row_o)) & 15) == 0 &&
      ((reinterpret_cast<uintptr_t>(cp) | reinterpret_cast<uintptr_t>(sp)) & 15) == 0) {
    const int sub = lane >> 3, j = lane & 7;
    float c[8], sn[8];
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cp + 8 * j);
    *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cp + 8 * j + 4);
    *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sp + 8 * j);
    *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sp + 8 * j + 4);
#pragma unroll 2
    for (int h0 = 0; h0 < heads; h0 += 4) {
      const int h = h0 + sub;
      const bool act = h < heads;
      V8 x1, x2, g1, g2;
#pragma unroll
      for (int e = 0; e < 8; ++e) x1.f[e] = 0.f, x2.f[e] = 0.f, g1.f[e] = 0.f, g2.f[e] = 0.f;
      if (act) {
        x1 = ld8(row_x + h * 128 + 8 * j);
        x2 = ld8(row_x + h * 128 + 64 + 8 * j);
        g1 = ld8(row_g + h * 128 + 8 * j);
        g2 = ld8(row_g + h * 128 + 64 + 8 * j);
      }
      float n1[8], n2[8], ss = 0.f, dot = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        n1[e] = scale * (g1.f[e] * c[e] - g2.f[e] * sn[e]);
        n2[e] = scale * (g1.f[e] * sn[e] + g2.f[e] * c[e]);
        ss += x1.f[e] * x1.f[e] + x2.f[e] * x2.f[e];
        dot += x1.f[e] * n1[e] + x2.f[e] * n2[e];
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        dot += __shfl_xor_sync(0xffffffffu, dot, o);
      }
      const float r = 1.0f / sqrtf(ss * inv_d + eps);
      const float coeff = r * r * r * dot * inv_d;
      if (act) {
        V8 o1, o2;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          o1.f[e] = r * n1[e] - coeff * x1.f[e];
          o2.f[e] = r * n2[e] - coeff * x2.f[e];
        }
        st8(row_o + h * 128 + 8 * j, o1);
        st8(row_o + h * 128 + 64 + 8 * j, o2);
      }
    }
    return;
  }
  const bool vec = (half % 2 == 0) && half <= 64 && (reinterpret_cast<uintptr_t>(cp) & 7) == 0 &&
                   (reinterpret_cast<uintptr_t>(sp) & 7) == 0 && (D % 2 == 0) &&
                   ((reinterpret_cast<uintptr_t>(row_x) | reinterpret_cast<uintptr_t>(row_g) |
                     reinterpret_cast<uintptr_t>(row_o)) & 3) == 0;
  if (vec) {
    const int d = lane * 2;
    const bool act = d < half;
    float cc[2] = {0.f, 0.f}, sc[2] = {0.f, 0.f};
    if (act) {
      const float2 c = *reinterpret_cast<const float2*>(cp + d);
      const float2 sn = *reinterpret_cast<const float2*>(sp + d);
      cc[0] = c.x, cc[1] = c.y, sc[0] = sn.x, sc[1] = sn.y;
    }
    for (int h = 0; h < heads; ++h) {
      const bf16* xp = row_x + h * D;
      const bf16* gp = row_g + h * D;
      bf16* op = row_o + h * D;
      float x1[2] = {0.f, 0.f}, x2[2] = {0.f, 0.f}, n1[2] = {0.f, 0.f}, n2[2] = {0.f, 0.f};
      if (act) {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(xp + d);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(xp + d + half);
        const __nv_bfloat162 ga = *reinterpret_cast<const __nv_bfloat162*>(gp + d);
        const __nv_bfloat162 gb = *reinterpret_cast<const __nv_bfloat162*>(gp + d + half);
        x1[0] = b2f(a.x), x1[1] = b2f(a.y), x2[0] = b2f(b.x), x2[1] = b2f(b.y);
        const float g1[2] = {b2f(ga.x), b2f(ga.y)}, g2[2] = {b2f(gb.x), b2f(gb.y)};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          n1[u] = scale * (g1[u] * cc[u] - g2[u] * sc[u]);
          n2[u] = scale * (g1[u] * sc[u] + g2[u] * cc[u]);
        }
      }
      const float ss = warp_sum(x1[0] * x1[0] + x1[1] * x1[1] + x2[0] * x2[0] + x2[1] * x2[1]);
      const float dot = warp_sum(x1[0] * n1[0] + x1[1] * n1[1] + x2[0] * n2[0] + x2[1] * n2[1]);
      const float r = 1.0f / sqrtf(ss * inv_d + eps);
      const float coeff = r * r * r * dot * inv_d;
      if (act) {
        *reinterpret_cast<__nv_bfloat162*>(op + d) =
            __floats2bfloat162_rn(r * n1[0] - coeff * x1[0], r * n1[1] - coeff * x1[1]);
        *reinterpret_cast<__nv_bfloat162*>(op + d + half) =
            __floats2bfloat162_rn(r * n2[0] - coeff * x2[0], r * n2[1] - coeff * x2[1]);
      }
    }
    return;
  }
  for (int h = 0; h < heads; ++h) {
    const bf16* xp = row_x + h * D;
    const bf16* gp = row_g + h * D;
    bf16* op = row_o + h * D;
    float ss = 0.0f, dot = 0.0f;
    for (int d = lane; d < half; d += 32) {
      const float c = cp[d], s = sp[d];
      const float x1 = b2f(xp[d]), x2 = b2f(xp[d + half]);
      const float g1 = b2f(gp[d]), g2 = b2f(gp[d + half]);
      ss += x1 * x1 + x2 * x2;
      dot += x1 * scale * (g1 * c - g2 * s) + x2 * scale * (g1 * s + g2 * c);
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float r = 1.0f / sqrtf(ss * inv_d + eps);
    const float coeff = r * r * r * dot * inv_d;
    for (int d = lane; d < half; d += 32) {
      const float c = cp[d], s = sp[d];
      const float x1 = b2f(xp[d]), x2 = b2f(xp[d + half]);
      const float g1 = b2f(gp[d]), g2 = b2f(gp[d + half]);
      op[d] = f2b(r * scale * (g1 * c - g2 * s) - coeff * x1);
      op[d + half] = f2b(r * scale * (g1 * s + g2 * c) - coeff * x2);
    }
  }
}

// ------------------------------------------------------------------ value gate
// Index checks of the gather/scatter kernels: `rows` > 0 is the size of the indexed table. An index outside it records
// kErrBadIndex in the status word (first error wins) and the caller skips the access.
__device__ __forceinline__ bool bad_index(int id, int rows, int* status) {
  if (rows <= 0 || (id >= 0 && id < rows)) return false;
  if (status != nullptr) atomicCAS(status, 0, 7 /* kErrBadIndex */);
  return true;
}
constexpr int kGateCh = 12;
__global__ void __launch_bounds__(kThreads) value_gate_fwd_kernel(const bf16* __restrict__ h, long long ldh,
                                                                  const bf16* __restrict__ ve,
                                                                  const bf16* __restrict__ gw, bf16* __restrict__ v,
                                                                  long long ldv, bf16* __restrict__ gate, int tokens,
                                                                  int KV, int D, const int* __restrict__ ids, int rows,
                                                                  int* status) {
  const long long wid = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (wid >= static_cast<long long>(tokens) * KV) return;
  const int lane = threadIdx.x & 31;
  const int tok = static_cast<int>(wid / KV), kh = static_cast<int>(wid % KV);
  float pre = 0.0f;
  if (lane < kGateCh) pre = b2f(h[static_cast<long long>(tok) * ldh + lane]) * b2f(gw[kh * kGateCh + lane]);
  pre = warp_sum(pre);
  const float g = 3.0f / (1.0f + __expf(-pre));
  if (lane == 0) gate[static_cast<long long>(tok) * KV + kh] = f2b(g);
  bf16* vp = v + static_cast<long long>(tok) * ldv + kh * D;
  if (ids != nullptr && bad_index(ids[tok], rows, status)) return;   // v stays as it was
  const bf16* ep = ve + (static_cast<long long>(ids ? ids[tok] : tok) * KV + kh) * D;
  for (int d = lane; d < D; d += 32) vp[d] = f2b(b2f(vp[d]) + g * b2f(ep[d]));
}

// dgw is reduced per block in shared memory, then with atomics.
__global__ void __launch_bounds__(kThreads) value_gate_bwd_kernel(
    const bf16* __restrict__ h, long long ldh, const bf16* __restrict__ ve, const bf16* __restrict__ gw,
    const bf16* __restrict__ gate, const bf16* __restrict__ dv, long long lddv, bf16* __restrict__ dve,
    float* __restrict__ dh12, float* __restrict__ dgw, int tokens, int KV, int D) {
  NC_DYNAMIC_SHARED(float, sh_dgw);  // KV*12
  for (int i = threadIdx.x; i < KV * kGateCh; i += blockDim.x) sh_dgw[i] = 0.0f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int tok = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (tok < tokens) {
    float dh_acc = 0.0f;  // lane j < 12 accumulates dh12[tok, j]
    const float hj = lane < kGateCh ? b2f(h[static_cast<long long>(tok) * ldh + lane]) : 0.0f;
    for (int kh = 0; kh < KV; ++kh) {
      const float g = b2f(gate[static_cast<long long>(tok) * KV + kh]);
      const bf16* dvp = dv + static_cast<long long>(tok) * lddv + kh * D;
      const bf16* ep = ve + (static_cast<long long>(tok) * KV + kh) * D;
      bf16* op = dve + (static_cast<long long>(tok) * KV + kh) * D;
      float dg = 0.0f;
      for (int d = lane; d < D; d += 32) {
        const float dvd = b2f(dvp[d]);
        dg += dvd * b2f(ep[d]);
        op[d] = f2b(g * dvd);
      }
      dg = warp_sum(dg);
      const float dpre = dg * g * (1.0f - g * (1.0f / 3.0f));
      if (lane < kGateCh) {
        atomicAdd(&sh_dgw[kh * kGateCh + lane], dpre * hj);
        dh_acc += dpre * b2f(gw[kh * kGateCh + lane]);
      }
    }
    if (lane < kGateCh) dh12[static_cast<long long>(tok) * kGateCh + lane] = dh_acc;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < KV * kGateCh; i += blockDim.x) atomicAdd(&dgw[i], sh_dgw[i]);
}

// 16-byte versions (D a multiple of 8 up to 128, aligned rows): a half-warp owns one (token, kv head) pair, each of
// its lanes one 8-element slice of the head, so a warp moves two heads per pass with every lane loading 16 bytes.
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// (Tried and dropped: issuing the embedding and value loads before the gate's own chain, and two or four pairs per
// half-warp with all loads up front: 0.100 - 0.109 ms against 0.096 for this form on the d20 shape; the extra registers
// cost more resident warps than the earlier loads gain.)
__global__ void __launch_bounds__(kThreads) value_gate_fwd_vec_kernel(const bf16* __restrict__ h, long long ldh,
                                                                      const bf16* __restrict__ ve,
                                                                      const bf16* __restrict__ gw, bf16* __restrict__ v,
                                                                      long long ldv, bf16* __restrict__ gate,
                                                                      int tokens, int KV, int D,
                                                                      const int* __restrict__ ids, int rows,
                                                                      int* status) {
  NC_PDL_PROLOGUE();
  const int lane = threadIdx.x & 31, li = lane & 15;
  const long long pair = (static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5)) * 2 + (lane >> 4);
  const bool valid = pair < static_cast<long long>(tokens) * KV;
  const int tok = valid ? static_cast<int>(pair / KV) : 0, kh = valid ? static_cast<int>(pair % KV) : 0;
  float pre = 0.0f;
  if (valid && li < kGateCh) pre = b2f(h[static_cast<long long>(tok) * ldh + li]) * b2f(gw[kh * kGateCh + li]);
  pre = half_warp_sum(pre);
  const float g = 3.0f / (1.0f + __expf(-pre));
  if (!valid) return;
  if (li == 0) gate[static_cast<long long>(tok) * KV + kh] = f2b(g);
  const int d = li * 8;
  if (d >= D) return;
  bf16* vp = v + static_cast<long long>(tok) * ldv + kh * D + d;
  // with `ids` the embedding rows are gathered from the table on the fly (decode: no separate gather pass)
  if (ids != nullptr && bad_index(ids[tok], rows, status)) return;
  const uint4 ev = *reinterpret_cast<const uint4*>(ve + (static_cast<long long>(ids ? ids[tok] : tok) * KV + kh) * D + d);
  const uint4 vv = *reinterpret_cast<const uint4*>(vp);
  const uint32_t ew[4] = {ev.x, ev.y, ev.z, ev.w}, vw[4] = {vv.x, vv.y, vv.z, vv.w};
  uint32_t o[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float lo = __uint_as_float(vw[e] << 16) + g * __uint_as_float(ew[e] << 16);
    const float hi = __uint_as_float(vw[e] & 0xffff0000u) + g * __uint_as_float(ew[e] & 0xffff0000u);
    const __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);
    o[e] = *reinterpret_cast<const uint32_t*>(&pk);
  }
  *reinterpret_cast<uint4*>(vp) = make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void __launch_bounds__(kThreads) value_gate_bwd_vec_kernel(
    const bf16* __restrict__ h, long long ldh, const bf16* __restrict__ ve, const bf16* __restrict__ gw,
    const bf16* __restrict__ gate, const bf16* __restrict__ dv, long long lddv, bf16* __restrict__ dve,
    float* __restrict__ dh12, float* __restrict__ dgw, int tokens, int KV, int D) {
  NC_DYNAMIC_SHARED(float, sh_dgw);  // KV*12
  for (int i = threadIdx.x; i < KV * kGateCh; i += blockDim.x) sh_dgw[i] = 0.0f;
  __syncthreads();
  const int lane = threadIdx.x & 31, li = lane & 15, half = lane >> 4;
  const int tok = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (tok < tokens) {
    float dh_acc = 0.0f;  // lane li < 12 of each half accumulates its heads' part of dh12[tok, li]
    const float hj = li < kGateCh ? b2f(h[static_cast<long long>(tok) * ldh + li]) : 0.0f;
    const int d = li * 8;
    // the loads of the next pair of heads are issued before this pair is reduced (two pairs in flight per lane)
    auto fetch = [&](int kh, uint4& dvv, uint4& ev, float& g) {
      dvv = make_uint4(0, 0, 0, 0);
      ev = make_uint4(0, 0, 0, 0);
      g = 0.0f;
      if (kh < KV) {
        g = b2f(gate[static_cast<long long>(tok) * KV + kh]);
        if (d < D) {
          dvv = *reinterpret_cast<const uint4*>(dv + static_cast<long long>(tok) * lddv + kh * D + d);
          ev = *reinterpret_cast<const uint4*>(ve + (static_cast<long long>(tok) * KV + kh) * D + d);
        }
      }
    };
    uint4 dvv_next, ev_next;
    float g_next;
    fetch(half, dvv_next, ev_next, g_next);
    for (int kh0 = 0; kh0 < KV; kh0 += 2) {
      const int kh = kh0 + half;
      const bool live = kh < KV;
      const uint4 dvv = dvv_next, ev = ev_next;
      const float g = g_next;
      fetch(kh + 2, dvv_next, ev_next, g_next);
      float dg = 0.0f;
      if (live) {
        if (d < D) {
          const uint32_t dw[4] = {dvv.x, dvv.y, dvv.z, dvv.w}, ew[4] = {ev.x, ev.y, ev.z, ev.w};
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float d0 = __uint_as_float(dw[e] << 16), d1 = __uint_as_float(dw[e] & 0xffff0000u);
            dg += d0 * __uint_as_float(ew[e] << 16) + d1 * __uint_as_float(ew[e] & 0xffff0000u);
            const __nv_bfloat162 pk = __floats2bfloat162_rn(g * d0, g * d1);
            o[e] = *reinterpret_cast<const uint32_t*>(&pk);
          }
          *reinterpret_cast<uint4*>(dve + (static_cast<long long>(tok) * KV + kh) * D + d) =
              make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      dg = half_warp_sum(dg);
      const float dpre = dg * g * (1.0f - g * (1.0f / 3.0f));
      if (live && li < kGateCh) {
        atomicAdd(&sh_dgw[kh * kGateCh + li], dpre * hj);
        dh_acc += dpre * b2f(gw[kh * kGateCh + li]);
      }
    }
    dh_acc += __shfl_xor_sync(0xffffffffu, dh_acc, 16);  // the two halves handled alternate heads
    if (lane < kGateCh) dh12[static_cast<long long>(tok) * kGateCh + lane] = dh_acc;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < KV * kGateCh; i += blockDim.x) atomicAdd(&dgw[i], sh_dgw[i]);
}

// ------------------------------------------------------------------ smear
constexpr int kSmearCh = 24;
__global__ void __launch_bounds__(kThreads) smear_fwd_kernel(const bf16* __restrict__ emb,
                                                             const bf16* __restrict__ gw, const float* lam,
                                                             const bf16* __restrict__ prev, bf16* __restrict__ x0,
                                                             float* __restrict__ sig, int tokens, int seq, int dim) {
  const int tok = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (tok >= tokens) return;
  const int lane = threadIdx.x & 31;
  const int t = tok % seq;
  const bf16* ep = emb + static_cast<long long>(tok) * dim;
  const bf16* pp = nullptr;
  if (t > 0) {
    pp = ep - dim;
  } else if (prev != nullptr) {
    pp = prev + static_cast<long long>(tok / seq) * dim;
  }
  float s = 0.0f;
  if (pp != nullptr) {
    float pre = lane < kSmearCh ? b2f(ep[lane]) * b2f(gw[lane]) : 0.0f;
    pre = warp_sum(pre);
    s = sigmoidf_(pre);
  }
  if (lane == 0) sig[tok] = s;
  const float g = (*lam) * s;
  bf16* op = x0 + static_cast<long long>(tok) * dim;
  for (int d = lane; d < dim; d += 32) {
    const float p = pp ? b2f(pp[d]) : 0.0f;
    op[d] = f2b(b2f(ep[d]) + g * p);
  }
}

__global__ void __launch_bounds__(kThreads) smear_bwd_kernel(const bf16* __restrict__ emb,
                                                             const bf16* __restrict__ gw, const float* lam,
                                                             const float* __restrict__ sig,
                                                             const bf16* __restrict__ dx0, bf16* __restrict__ de,
                                                             float* __restrict__ dgw24, float* __restrict__ dlam,
                                                             int tokens, int seq, int dim) {
  __shared__ float sh_gw[kSmearCh];
  __shared__ float sh_lam;
  if (threadIdx.x < kSmearCh) sh_gw[threadIdx.x] = 0.0f;
  if (threadIdx.x == 0) sh_lam = 0.0f;
  __syncthreads();
  const int tok = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (tok < tokens) {
    const int t = tok % seq;
    const float lambda = *lam;
    const bf16* ep = emb + static_cast<long long>(tok) * dim;
    const bf16* dp = dx0 + static_cast<long long>(tok) * dim;
    bf16* op = de + static_cast<long long>(tok) * dim;
    float dpre = 0.0f;
    if (t > 0) {
      float dg = 0.0f;
      for (int d = lane; d < dim; d += 32) dg += b2f(dp[d]) * b2f(ep[d - dim]);
      dg = warp_sum(dg);
      const float s = sig[tok];
      dpre = dg * lambda * s * (1.0f - s);
      if (lane == 0) atomicAdd(&sh_lam, dg * s);
      if (lane < kSmearCh) atomicAdd(&sh_gw[lane], dpre * b2f(ep[lane]));
    }
    const bool tail = t == seq - 1;
    const float gnext = tail ? 0.0f : lambda * sig[tok + 1];
    for (int d = lane; d < dim; d += 32) {
      float v = b2f(dp[d]);
      if (d < kSmearCh) v += dpre * b2f(gw[d]);
      if (!tail) v += gnext * b2f(dp[d + dim]);
      op[d] = f2b(v);
    }
  }
  __syncthreads();
  if (threadIdx.x < kSmearCh) atomicAdd(&dgw24[threadIdx.x], sh_gw[threadIdx.x]);
  if (threadIdx.x == 0) atomicAdd(dlam, sh_lam);
}

// ------------------------------------------------------------------ embeddings
__global__ void __launch_bounds__(kThreads) embedding_fwd_kernel(const int* __restrict__ ids,
                                                                 const bf16* __restrict__ table,
                                                                 bf16* __restrict__ out, int tokens, int dim,
                                                                 int rows, int* status) {
  const int tok = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (tok >= tokens) return;
  const int lane = threadIdx.x & 31;
  bf16* dst = out + static_cast<long long>(tok) * dim;
  if (bad_index(ids[tok], rows, status)) {   // an id outside the table: a zero row, and the status word says so
    for (int i = lane; i < dim; i += 32) dst[i] = f2b(0.0f);
    return;
  }
  const bf16* src = table + static_cast<long long>(ids[tok]) * dim;
  if (dim % 8 == 0 && aligned16(src) && aligned16(dst)) {
    for (int i = lane * 8; i < dim; i += 256) *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
  } else {
    for (int i = lane; i < dim; i += 32) dst[i] = src[i];
  }
}

__global__ void __launch_bounds__(kThreads) embedding_bwd_kernel(const int* __restrict__ ids,
                                                                 const bf16* __restrict__ dout, long long ld,
                                                                 float* __restrict__ dtable, int tokens, int dim,
                                                                 int rows, int* status) {
  const int tok = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (tok >= tokens) return;
  if (bad_index(ids[tok], rows, status)) return;
  const int lane = threadIdx.x & 31;
  const bf16* src = dout + static_cast<long long>(tok) * ld;
  float* dst = dtable + static_cast<long long>(ids[tok]) * dim;
  if (dim % 4 == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    for (int i = lane * 4; i < dim; i += 128) {
      const float a = b2f(src[i]), b = b2f(src[i + 1]), c = b2f(src[i + 2]), d = b2f(src[i + 3]);
#ifdef NC_EMU
      atomicAdd(dst + i, a), atomicAdd(dst + i + 1, b), atomicAdd(dst + i + 2, c), atomicAdd(dst + i + 3, d);
#else
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + i), "f"(a), "f"(b), "f"(c), "f"(d)
                   : "memory");
#endif
    }
  } else {
    for (int i = lane; i < dim; i += 32) atomicAdd(dst + i, b2f(src[i]));
  }
}

// Deterministic variant: the token ids arrive stably sorted (`perm[j]` = original row of sorted position j). The
// warp at the head of a run of equal ids sums the run's rows in ascending row order in fp32 registers and is the
// only writer of that table row, so the result does not depend on scheduling (the atomic kernel above adds in
// arrival order). The reference's embedding backward is deterministic too, one thread per (row of the table,
// column) scanning all tokens (backends/cuda/kernels/embedding.cu); this keeps that property at O(tokens) work.
__global__ void __launch_bounds__(kThreads) embedding_bwd_sorted_kernel(const int* __restrict__ sorted_ids,
                                                                        const int* __restrict__ perm,
                                                                        const bf16* __restrict__ dout, long long ld,
                                                                        float* __restrict__ dtable, int tokens,
                                                                        int dim, int rows, int* status) {
  const int i = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (i >= tokens) return;
  const int id = sorted_ids[i];
  if (i > 0 && sorted_ids[i - 1] == id) return;  // not the head of its run
  if (bad_index(id, rows, status)) return;
  const int lane = threadIdx.x & 31;
  float* dst = dtable + static_cast<long long>(id) * dim;
  const bool vec = dim % 8 == 0 && ld % 8 == 0 && aligned16(dout) && aligned16(dst);
  if (vec) {
    for (int c0 = lane * 8; c0 < dim; c0 += 256) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = i; j < tokens && sorted_ids[j] == id; ++j) {
        const uint4 v = *reinterpret_cast<const uint4*>(dout + static_cast<long long>(perm[j]) * ld + c0);
        const bf16* h = reinterpret_cast<const bf16*>(&v);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += b2f(h[k]);
      }
      float4* d4 = reinterpret_cast<float4*>(dst + c0);
      float4 lo = d4[0], hi = d4[1];
      lo.x += acc[0], lo.y += acc[1], lo.z += acc[2], lo.w += acc[3];
      hi.x += acc[4], hi.y += acc[5], hi.z += acc[6], hi.w += acc[7];
      d4[0] = lo, d4[1] = hi;
    }
  } else {
    for (int c = lane; c < dim; c += 32) {
      float acc = 0.f;
      for (int j = i; j < tokens && sorted_ids[j] == id; ++j) acc += b2f(dout[static_cast<long long>(perm[j]) * ld + c]);
      dst[c] += acc;
    }
  }
}

// ------------------------------------------------------------------ softcap + cross entropy (+ backward, in place)
__device__ __forceinline__ float tanh_acc(float x) {
  // 1 - 2/(exp(2x)+1): accurate to a few ulp and saturates cleanly for large |x|
  const float e = __expf(2.0f * x);
  return 1.0f - 2.0f / (e + 1.0f);
}

__global__ void __launch_bounds__(256) classifier_kernel(bf16* __restrict__ logits, long long ld,
                                                         const int* __restrict__ targets, float* __restrict__ losses,
                                                         const float* __restrict__ row_scale,
                                                         const float* __restrict__ dlogit_scale, int rows, int vocab,
                                                         int padded, float softcap, int ignore_index, bool want_grad,
                                                         int* status) {
  __shared__ float sh[32];
  const int row = blockIdx.x;
  bf16* lp = logits + static_cast<long long>(row) * ld;
  int target = targets[row];
  if (target != ignore_index && (target < 0 || target >= vocab)) {   // not a class: counted as ignored, and reported
    if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, 7 /* kErrBadIndex */);
    target = ignore_index;
  }
  const float inv_cap = 1.0f / softcap;
  const bool vec = (vocab % 8 == 0) && (padded % 8 == 0) && aligned16(lp) && (ld % 8 == 0);
  if (target == ignore_index) {
    if (threadIdx.x == 0) losses[row] = 0.0f;
    if (want_grad) {
      for (int i = threadIdx.x; i < padded; i += blockDim.x) lp[i] = f2b(0.0f);
    }
    return;
  }
  // read before the gradient pass of any warp can overwrite it (see classifier_smem_kernel)
  const float target_logit = threadIdx.x == 0 ? b2f(lp[target]) : 0.0f;
  // pass 1: online max / sum of exp over the capped logits
  float m = -CUDART_INF_F, l = 0.0f;
  if (vec) {
    for (int i = threadIdx.x * 8; i < vocab; i += blockDim.x * 8) {
      const V8 v = ld8(lp + i);
      float z[8], cm = m;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        z[e] = softcap * tanh_acc(v.f[e] * inv_cap);
        cm = fmaxf(cm, z[e]);
      }
      float add = 0.0f;
#pragma unroll
      for (int e = 0; e < 8; ++e) add += __expf(z[e] - cm);
      l = l * __expf(m - cm) + add;
      m = cm;
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float z = softcap * tanh_acc(b2f(lp[i]) * inv_cap);
      const float cm = fmaxf(m, z);
      l = l * __expf(m - cm) + __expf(z - cm);
      m = cm;
    }
  }
  // block combine of (m, l)
  float bm = warp_max(m);
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) sh[warp] = bm;
    __syncthreads();
    float t = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : -CUDART_INF_F;
    if (warp == 0) t = warp_max(t);
    if (threadIdx.x == 0) sh[0] = t;
    __syncthreads();
    bm = sh[0];
    __syncthreads();
  }
  const float lsum = block_sum(m == -CUDART_INF_F ? 0.0f : l * __expf(m - bm), sh);
  if (threadIdx.x == 0) {
    const float tz = softcap * tanh_acc(target_logit * inv_cap);
    losses[row] = logf(lsum) + bm - tz;
  }
  if (!want_grad) return;
  __syncthreads();  // the target logit was read above, before anything is overwritten
  const float inv = 1.0f / lsum;
  const float scale = *dlogit_scale;
  const float rs = row_scale ? row_scale[row] : 1.0f;
  if (vec) {
    for (int i = threadIdx.x * 8; i < padded; i += blockDim.x * 8) {
      V8 o;
      if (i < vocab) {
        const V8 v = ld8(lp + i);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float t = tanh_acc(v.f[e] * inv_cap);
          const float p = __expf(softcap * t - bm) * inv;
          const float onehot = (i + e == target) ? 1.0f : 0.0f;
          // rounded once before the loss scale, as the two-pass definition does
          o.f[e] = b2f(f2b((p - onehot) * (1.0f - t * t) * rs)) * scale;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) o.f[e] = 0.0f;
      }
      st8(lp + i, o);
    }
  } else {
    for (int i = threadIdx.x; i < padded; i += blockDim.x) {
      float o = 0.0f;
      if (i < vocab) {
        const float t = tanh_acc(b2f(lp[i]) * inv_cap);
        const float p = __expf(softcap * t - bm) * inv;
        const float onehot = (i == target) ? 1.0f : 0.0f;
        o = b2f(f2b((p - onehot) * (1.0f - t * t) * rs)) * scale;
      }
      lp[i] = f2b(o);
    }
  }
}

// One CTA per row with the row's logits kept in shared memory between the two sweeps, so a chunk of logits is
// read from HBM once and written once. The soft cap bounds every logit to [-cap, cap], which makes the running
// maximum unnecessary: exp(z - cap) cannot overflow and its sum over any vocabulary stays far above the fp32
// denormal range. tanh is the single-instruction approximation (relative error 2^-11, four times finer than the
// bf16 rounding of its input). Per element: tanh + ex2 in each sweep.
#ifdef NC_EMU
__device__ __forceinline__ float tanh_fast(float x) { return std::tanh(x); }
__device__ __forceinline__ float ex2_fast(float x) { return std::exp2(x); }
__device__ __forceinline__ float lg2_fast(float x) { return std::log2(x); }
#else
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2_fast(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
#endif

constexpr int kClsThreads = 512;

// STAGE: the row is parked in shared memory between the two passes (one CTA per SM for a 64K-entry row). Without it
// the second pass reads the row again through L2, where the first pass left it, and several CTAs share an SM, so one
// CTA's exponentials overlap another's loads and stores.
// CACHE (without STAGE, gradient wanted): the first sweep writes e = exp(z - cap) back over the logit it came from,
// as bf16, and the second sweep rebuilds both factors of the gradient from it: p = e / sum and, since
// log2(e) = cap * log2(e) * (t - 1), 1 - t = -log2(e) / c2 and 1 - t^2 = (1 - t)(1 + t). That is one lg2 in place of
// a tanh and an ex2: three special-function operations per logit instead of four, on a kernel that is bound by that
// unit. The row stays in L2 between the sweeps either way; the extra store of the first sweep is overwritten by the
// gradient before it has to leave L2. e carries bf16 rounding (2^-9 relative) into p, of the size of the rounding the
// gradient itself gets; 1 - t comes out with an absolute error of about 1e-4.
template <bool STAGE, bool CACHE = false>
__global__ void __launch_bounds__(kClsThreads) classifier_smem_kernel(
    bf16* __restrict__ logits, long long ld, const int* __restrict__ targets, float* __restrict__ losses,
    const float* __restrict__ row_scale, const float* __restrict__ dlogit_scale, int vocab, int padded,
    float softcap, int ignore_index, bool want_grad, int* status) {
  NC_DYNAMIC_SHARED(unsigned char, cls_smem);
  bf16* row_s = reinterpret_cast<bf16*>(cls_smem);
  __shared__ float sh[32];
  const int row = blockIdx.x;
  bf16* lp = logits + static_cast<long long>(row) * ld;
  int target = targets[row];
  if (target != ignore_index && (target < 0 || target >= vocab)) {
    if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, 7 /* kErrBadIndex */);
    target = ignore_index;
  }
  if (target == ignore_index) {
    if (threadIdx.x == 0) losses[row] = 0.0f;
    if (want_grad) {
      for (int i = threadIdx.x * 8; i < padded; i += kClsThreads * 8)
        *reinterpret_cast<uint4*>(lp + i) = make_uint4(0, 0, 0, 0);
    }
    return;
  }
  const float inv_cap = 1.0f / softcap;
  const float c2 = softcap * 1.4426950408889634f;  // cap * log2(e): exp(z - cap) = 2^(c2 * (t - 1))
  // The target's logit is read here, before anything is written: after the block-wide sum other warps go straight
  // on to overwrite the row with its gradient, and a read at that point would race with the thread that owns
  // the target's position.
  // (With CACHE the first sweep overwrites the row itself, so there the thread that owns the target's vector hands
  // its logit over through shared memory.)
  __shared__ float sh_target;
  float target_logit = (!CACHE && threadIdx.x == 0) ? b2f(lp[target]) : 0.0f;
  const bool cache = CACHE && want_grad;
  float l = 0.0f;
  // four 16-byte loads per thread are issued before any of them is used: 32 KB in flight per CTA
  constexpr int kBatch = 4;
  for (int i0 = threadIdx.x * 8; i0 < vocab; i0 += kClsThreads * 8 * kBatch) {
    uint4 raw[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = i0 + u * kClsThreads * 8;
      raw[u] = i >= vocab ? make_uint4(0, 0, 0, 0)
                          : STAGE ? __ldcs(reinterpret_cast<const uint4*>(lp + i))
                                  : *reinterpret_cast<const uint4*>(lp + i);
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = i0 + u * kClsThreads * 8;
      if (i >= vocab) break;
      if (STAGE && want_grad) *reinterpret_cast<uint4*>(row_s + i) = raw[u];
      const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
      if (CACHE && static_cast<unsigned>(target - i) < 8u) {
        const uint32_t tw = w[(target - i) >> 1];
        sh_target = __uint_as_float(((target - i) & 1) ? (tw & 0xffff0000u) : (tw << 16));
      }
      uint32_t packed[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float t0 = tanh_fast(__uint_as_float(w[e] << 16) * inv_cap);
        const float t1 = tanh_fast(__uint_as_float(w[e] & 0xffff0000u) * inv_cap);
        const float e0 = ex2_fast(fmaf(c2, t0, -c2)), e1 = ex2_fast(fmaf(c2, t1, -c2));
        l += e0 + e1;
        if (CACHE) {
          const __nv_bfloat162 pk = __floats2bfloat162_rn(e0, e1);
          packed[e] = *reinterpret_cast<const uint32_t*>(&pk);
        }
      }
      if (cache) *reinterpret_cast<uint4*>(lp + i) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
  }
  const float lsum = block_sum(l, sh);
  if (CACHE) target_logit = sh_target;  // written before the barriers of block_sum
  if (threadIdx.x == 0) losses[row] = logf(lsum) + softcap - softcap * tanh_fast(target_logit * inv_cap);
  if (!want_grad) return;  // block_sum ended with a barrier: every thread's part of the row is in shared memory
  const float inv = 1.0f / lsum;
  const float neg_inv_c2 = -1.0f / c2;
  const float scale = *dlogit_scale;
  const float rs = row_scale ? row_scale[row] : 1.0f;
  for (int i = threadIdx.x * 8; i < padded; i += kClsThreads * 8) {
    uint4 outv = make_uint4(0, 0, 0, 0);
    if (i < vocab) {
      const uint4 raw = STAGE ? *reinterpret_cast<const uint4*>(row_s + i) : *reinterpret_cast<const uint4*>(lp + i);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float p0, p1, d0, d1;  // probability and 1 - t^2
        if (CACHE) {
          const float e0 = __uint_as_float(w[e] << 16), e1 = __uint_as_float(w[e] & 0xffff0000u);
          const float s0 = lg2_fast(e0) * neg_inv_c2, s1 = lg2_fast(e1) * neg_inv_c2;  // 1 - t
          p0 = e0 * inv, p1 = e1 * inv;
          d0 = s0 * (2.0f - s0), d1 = s1 * (2.0f - s1);
        } else {
          const float t0 = tanh_fast(__uint_as_float(w[e] << 16) * inv_cap);
          const float t1 = tanh_fast(__uint_as_float(w[e] & 0xffff0000u) * inv_cap);
          p0 = ex2_fast(fmaf(c2, t0, -c2)) * inv, p1 = ex2_fast(fmaf(c2, t1, -c2)) * inv;
          d0 = 1.0f - t0 * t0, d1 = 1.0f - t1 * t1;
        }
        const float h0 = (i + 2 * e == target) ? 1.0f : 0.0f;
        const float h1 = (i + 2 * e + 1 == target) ? 1.0f : 0.0f;
        // rounded once before the loss scale, as the two-pass definition does
        const float g0 = b2f(f2b((p0 - h0) * d0 * rs)) * scale;
        const float g1 = b2f(f2b((p1 - h1) * d1 * rs)) * scale;
        const __nv_bfloat162 pk = __floats2bfloat162_rn(g0, g1);
        o[e] = *reinterpret_cast<const uint32_t*>(&pk);
      }
      outv = make_uint4(o[0], o[1], o[2], o[3]);
    }
    *reinterpret_cast<uint4*>(lp + i) = outv;
  }
}

// ------------------------------------------------------------------ gradient norm
// Sum of squares of an fp32 span in fp64. Each thread keeps eight 16-byte loads in flight, squares and adds their 32
// values in fp32 (four partial sums of eight terms) and only then touches the fp64 accumulator, so the conversion and
// the double add are rare. Six blocks of 256 threads are resident per SM (the register bound asks for at most 42):
// about 190 KB in flight per SM, which is what HBM latency needs; the grid is exactly the resident blocks.
constexpr int kSumsqBlocksPerSm = 6;
__global__ void __launch_bounds__(256, kSumsqBlocksPerSm) sumsq_kernel(const float* __restrict__ g, long long n,
                                                                       double* out) {
  __shared__ double shd[8];
  double acc = 0.0;
  const long long nv = n / 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  constexpr int U = 8;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < nv; i0 += stride * U) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      v[u] = i < nv ? g4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int u = 0; u < U; ++u) part[u & 3] += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
    acc += static_cast<double>(part[0] + part[1]) + static_cast<double>(part[2] + part[3]);
  }
  if (blockIdx.x == 0) {
    for (long long i = nv * 4 + threadIdx.x; i < n; i += blockDim.x) acc += static_cast<double>(g[i]) * g[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) shd[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < 8; ++w) t += shd[w];
    atomicAdd(out, t);
  }
}

__global__ void finish_norm_kernel(const double* sumsq, float clip, float* norm_clip) {
  const float norm = static_cast<float>(sqrt(*sumsq));
  norm_clip[0] = norm;
  norm_clip[1] = (clip > 0.0f && norm > clip) ? clip / norm : 1.0f;
}

inline int flat_grid(long long n) {
  long long b = (n / 8 + 255) / 256;
  if (b < 1) b = 1;
  if (b > 148 * 8) b = 148 * 8;
  return static_cast<int>(b);
}

}  // namespace

// ------------------------------------------------------------------ launchers
#ifndef NC_EMU
void rmsnorm_fwd(const bf16* x, long long ldx, bf16* y, float* rstd, int rows, int dim, float eps, cudaStream_t s,
                 uint8_t* yq, uint8_t* sf) {
  if (rows <= 0) return;
  launch_maybe_pdl(rmsnorm_kernel<0>, dim3(blocks_for_rows(rows)), dim3(kThreads), 0, s, x, ldx, nullptr, nullptr, nullptr,
                   nullptr, y, rstd, rows, dim, eps, yq, sf);
}
void rmsnorm_apply(const bf16* x, long long ldx, const float* rstd, bf16* y, int rows, int dim, cudaStream_t s) {
  if (rows <= 0) return;
  rmsnorm_kernel<1><<<blocks_for_rows(rows), kThreads, 0, s>>>(x, ldx, nullptr, nullptr, nullptr, nullptr, y,
                                                               const_cast<float*>(rstd), rows, dim, 0.0f);
}
void rmsnorm_bwd(const bf16* x, const bf16* dy, const float* rstd, const bf16* residual, bf16* dx, int rows, int dim,
                 cudaStream_t s) {
  if (rows <= 0) return;
  rmsnorm_bwd_kernel<<<blocks_for_rows(rows), kThreads, 0, s>>>(x, dy, rstd, residual, dx, rows, dim);
}
void blend_norm_fwd(const bf16* x, const bf16* x0, const float* lam_r, const float* lam_0, bf16* xr, bf16* h,
                    float* rstd, int rows, int dim, float eps, cudaStream_t s, uint8_t* hq, uint8_t* sf) {
  if (rows <= 0) return;
  launch_maybe_pdl(rmsnorm_kernel<2>, dim3(blocks_for_rows(rows)), dim3(kThreads), 0, s, x, static_cast<long long>(dim),
                   x0, lam_r, lam_0, xr, h, rstd, rows, dim, eps, hq, sf);
}
const char* norm_blend_bwd(const bf16* xr, const bf16* dh, const float* rstd, const bf16* residual, const float* extra,
                           int extra_cols, const bf16* x, const bf16* x0, const float* lam_r, const float* lam_0, bf16* dx,
                           bf16* dx0, bool accumulate_dx0, float* g_lam_r, float* g_lam_0, int rows, int dim,
                           cudaStream_t s) {
  if (rows <= 0) return nullptr;
  if (dim % 8 != 0 || !aligned16(xr) || !aligned16(dh) || !aligned16(residual) || !aligned16(x) || !aligned16(x0) ||
      !aligned16(dx) || !aligned16(dx0))
    return "norm_blend_bwd: rows must be multiples of 8 elements and 16-byte aligned";
  if (extra != nullptr && (extra_cols <= 0 || extra_cols > dim)) return "norm_blend_bwd: bad extra column count";
  norm_blend_bwd_kernel<<<blocks_for_rows(rows), kThreads, 0, s>>>(xr, dh, rstd, residual, extra, extra_cols, x, x0, lam_r,
                                                                 lam_0, dx, dx0, accumulate_dx0 ? 1 : 0, g_lam_r, g_lam_0,
                                                                 rows, dim);
  return nullptr;
}
void blend_bwd(const bf16* dxr, const bf16* x, const bf16* x0, const float* lam_r, const float* lam_0, bf16* dx,
               bf16* dx0, bool accumulate_dx0, float* dlam2, long long n, cudaStream_t s) {
  flat_kernel<0><<<flat_grid(n), 256, 0, s>>>(dxr, x, x0, lam_r, lam_0, dx, dx0, accumulate_dx0 ? 1 : 0, dlam2, n);
}
void backout_fwd(const bf16* x, const bf16* xb, const float* lam, bf16* y, long long n, cudaStream_t s) {
  flat_kernel<1><<<flat_grid(n), 256, 0, s>>>(x, xb, nullptr, lam, nullptr, y, nullptr, 0, nullptr, n);
}
void backout_bwd(const bf16* dy, const bf16* xb, const float* lam, bf16* dxb, float* dlam, long long n,
                 cudaStream_t s) {
  flat_kernel<2><<<flat_grid(n), 256, 0, s>>>(dy, xb, nullptr, lam, nullptr, dxb, nullptr, 0, dlam, n);
}
void add_bf16(const bf16* a, const bf16* b, bf16* out, long long n, cudaStream_t s) {
  flat_kernel<3><<<flat_grid(n), 256, 0, s>>>(a, b, nullptr, nullptr, nullptr, out, nullptr, 0, nullptr, n);
}
void add_cols(bf16* dh, long long ld, const float* extra, int rows, int ncols, cudaStream_t s) {
  const int n = rows * ncols;
  if (n <= 0) return;
  add_cols_kernel<<<(n + 255) / 256, 256, 0, s>>>(dh, ld, extra, rows, ncols);
}
void qk_prep_fwd(const bf16* in, long long ld_in, bf16* out, long long ld_out, const float* cos, const float* sin,
                 const int* positions, int tokens, int seq, int heads, int D, float eps, float scale, cudaStream_t s) {
  if (tokens <= 0 || heads <= 0) return;
  qk_prep_fwd_kernel<<<blocks_for_rows(tokens), kThreads, 0, s>>>(in, ld_in, out, ld_out, cos, sin, positions, tokens, seq,
                                                             heads, D, eps, scale);
}
void qk_prep_bwd(const bf16* pre, long long ld_pre, const bf16* grad, long long ld_grad, bf16* out, long long ld_out,
                 const float* cos, const float* sin, int tokens, int seq, int heads, int D, float eps, float scale,
                 cudaStream_t s) {
  if (tokens <= 0 || heads <= 0) return;
  qk_prep_bwd_kernel<<<blocks_for_rows(tokens), kThreads, 0, s>>>(pre, ld_pre, grad, ld_grad, out, ld_out, cos, sin, tokens,
                                                             seq, heads, D, eps, scale);
}
void value_gate_fwd(const bf16* h, long long ldh, const bf16* ve, const bf16* gate_w, bf16* v, long long ldv,
                    bf16* gate, int tokens, int KV, int D, cudaStream_t s, const int* ids, int rows, int* status) {
  const long long n = static_cast<long long>(tokens) * KV;
  if (n <= 0) return;
  if (D % 8 == 0 && D <= 128 && ldv % 8 == 0 && aligned16(v) && aligned16(ve)) {
    launch_maybe_pdl(value_gate_fwd_vec_kernel, dim3(blocks_for_rows((n + 1) / 2)), dim3(kThreads), 0, s, h, ldh, ve,
                     gate_w, v, ldv, gate, tokens, KV, D, ids, rows, status);
    return;
  }
  value_gate_fwd_kernel<<<blocks_for_rows(n), kThreads, 0, s>>>(h, ldh, ve, gate_w, v, ldv, gate, tokens, KV, D, ids,
                                                                rows, status);
}
void value_gate_bwd(const bf16* h, long long ldh, const bf16* ve, const bf16* gate_w, const bf16* gate, const bf16* dv,
                    long long lddv, bf16* dve, float* dh12, float* dgw, int tokens, int KV, int D, cudaStream_t s) {
  if (tokens <= 0) return;
  if (D % 8 == 0 && D <= 128 && lddv % 8 == 0 && aligned16(dv) && aligned16(ve) && aligned16(dve)) {
    value_gate_bwd_vec_kernel<<<blocks_for_rows(tokens), kThreads, KV * kGateCh * sizeof(float), s>>>(
        h, ldh, ve, gate_w, gate, dv, lddv, dve, dh12, dgw, tokens, KV, D);
    return;
  }
  value_gate_bwd_kernel<<<blocks_for_rows(tokens), kThreads, KV * kGateCh * sizeof(float), s>>>(
      h, ldh, ve, gate_w, gate, dv, lddv, dve, dh12, dgw, tokens, KV, D);
}
void smear_fwd(const bf16* emb, const bf16* gate_w, const float* lam, const bf16* prev, bf16* x0, float* sig,
               int tokens, int seq, int dim, cudaStream_t s) {
  if (tokens <= 0) return;
  smear_fwd_kernel<<<blocks_for_rows(tokens), kThreads, 0, s>>>(emb, gate_w, lam, prev, x0, sig, tokens, seq, dim);
}
void smear_bwd(const bf16* emb, const bf16* gate_w, const float* lam, const float* sig, const bf16* dx0, bf16* de,
               float* dgw24, float* dlam, int tokens, int seq, int dim, cudaStream_t s) {
  if (tokens <= 0) return;
  smear_bwd_kernel<<<blocks_for_rows(tokens), kThreads, 0, s>>>(emb, gate_w, lam, sig, dx0, de, dgw24, dlam, tokens,
                                                                seq, dim);
}
void embedding_fwd(const int* ids, const bf16* table, bf16* out, int tokens, int dim, cudaStream_t s, int rows,
                   int* status) {
  if (tokens <= 0) return;
  embedding_fwd_kernel<<<blocks_for_rows(tokens), kThreads, 0, s>>>(ids, table, out, tokens, dim, rows, status);
}
void embedding_bwd(const int* ids, const bf16* dout, long long ld, float* dtable, int tokens, int dim, cudaStream_t s,
                   int rows, int* status) {
  if (tokens <= 0) return;
  embedding_bwd_kernel<<<blocks_for_rows(tokens), kThreads, 0, s>>>(ids, dout, ld, dtable, tokens, dim, rows, status);
}
void embedding_bwd_sorted(const int* sorted_ids, const int* perm, const bf16* dout, long long ld, float* dtable,
                          int tokens, int dim, cudaStream_t s, int rows, int* status) {
  if (tokens <= 0) return;
  embedding_bwd_sorted_kernel<<<blocks_for_rows(tokens), kThreads, 0, s>>>(sorted_ids, perm, dout, ld, dtable, tokens,
                                                                           dim, rows, status);
}
void classifier_fwd_bwd(bf16* logits, long long ld, const int* targets, float* losses, const float* row_scale,
                        const float* dlogit_scale, int rows, int vocab, int padded, float softcap, int ignore_index,
                        bool want_grad, cudaStream_t s, int* status) {
  if (rows <= 0) return;
  const size_t row_bytes = static_cast<size_t>(padded) * sizeof(bf16);
  const bool vec = vocab % 8 == 0 && padded % 8 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
  static const bool stage = [] {
    const char* e = getenv("NANOCHAT_CLS_STAGE");
    return e != nullptr && e[0] == '1';
  }();
  static const bool cache = [] {
    const char* e = getenv("NANOCHAT_CLS_CACHE");
    return e == nullptr || e[0] != '0';
  }();
  if (vec && !stage) {
    if (cache && want_grad)
      classifier_smem_kernel<false, true><<<rows, kClsThreads, 0, s>>>(
          logits, ld, targets, losses, row_scale, dlogit_scale, vocab, padded, softcap, ignore_index, want_grad, status);
    else
      classifier_smem_kernel<false><<<rows, kClsThreads, 0, s>>>(logits, ld, targets, losses, row_scale, dlogit_scale,
                                                                 vocab, padded, softcap, ignore_index, want_grad, status);
    return;
  }
  if (vec && row_bytes <= 200 * 1024) {
    cudaFuncSetAttribute(classifier_smem_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    classifier_smem_kernel<true><<<rows, kClsThreads, want_grad ? row_bytes : 0, s>>>(
        logits, ld, targets, losses, row_scale, dlogit_scale, vocab, padded, softcap, ignore_index, want_grad, status);
    return;
  }
  classifier_kernel<<<rows, 256, 0, s>>>(logits, ld, targets, losses, row_scale, dlogit_scale, rows, vocab, padded,
                                         softcap, ignore_index, want_grad, status);
}
void sumsq_f32(const float* g, long long n, double* out, cudaStream_t s) {
  if (n <= 0) return;
  long long b = (n / 4 + 255) / 256;
  if (b < 1) b = 1;
  // a grid of exactly the resident blocks, each striding over the span, has no partial last wave
  if (b > 148 * kSumsqBlocksPerSm) b = 148 * kSumsqBlocksPerSm;
  sumsq_kernel<<<static_cast<int>(b), 256, 0, s>>>(g, n, out);
}
void finish_norm(const double* sumsq, float clip, float* norm_clip, cudaStream_t s) {
  finish_norm_kernel<<<1, 1, 0, s>>>(sumsq, clip, norm_clip);
}

#endif  // !NC_EMU

}  // namespace nc

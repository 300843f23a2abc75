// Optimizer kernels: fused AdamW, and the elementwise stages of Muon around its tensor-core products.
// The reference runs Muon as 39 launches per shape group with 17 small kernels
// (backends/cuda/kernels/muon.cu:83-464); here the momentum / Nesterov / row-norm stage, the row
// rescale + bf16 cast, and the NorMuon-scaled cautious update are one kernel each, and the Polar
// Express products run on the tcgen05 GEMM (batched over the matrices of a group).
#include "host_build.h"

#include "optim.h"

#include <stdint.h>

namespace nc {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ value,
                                                    const float* __restrict__ grad, float* __restrict__ m,
                                                    float* __restrict__ v, long long n, float lr, float beta1,
                                                    float beta2, float eps, float wd, float inv_bias2,
                                                    float step_size, const float* grad_scale) {
  const float gs = grad_scale ? *grad_scale : 1.0f;
  const float decay = 1.0f - lr * wd;
  const long long nv = n / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(master)[i];
    const float4 g4 = reinterpret_cast<const float4*>(grad)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float pp[4] = {p.x, p.y, p.z, p.w};
    const float gg[4] = {g4.x, g4.y, g4.z, g4.w};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float g = gg[e] * gs;
      float pi = pp[e] * decay;
      mm[e] = mm[e] + (1.0f - beta1) * (g - mm[e]);
      vv[e] = vv[e] + (1.0f - beta2) * (g * g - vv[e]);
      const float denom = sqrtf(vv[e] * inv_bias2) + eps;
      pi -= step_size * (mm[e] / denom);
      pp[e] = pi;
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (value != nullptr) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]);
      __nv_bfloat162 hi = __floats2bfloat162_rn(pp[2], pp[3]);
      uint2 w;
      w.x = *reinterpret_cast<uint32_t*>(&lo);
      w.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(value)[i] = w;
    }
  }
  if (blockIdx.x == 0) {
    for (long long i = nv * 4 + threadIdx.x; i < n; i += blockDim.x) {
      const float g = grad[i] * gs;
      float pi = master[i] * decay;
      const float mi = m[i] + (1.0f - beta1) * (g - m[i]);
      const float vi = v[i] + (1.0f - beta2) * (g * g - v[i]);
      m[i] = mi;
      v[i] = vi;
      pi -= step_size * (mi / (sqrtf(vi * inv_bias2) + eps));
      master[i] = pi;
      if (value != nullptr) value[i] = __float2bfloat16_rn(pi);
    }
  }
}

// one warp per row
__global__ void __launch_bounds__(256) muon_nesterov_kernel(const float* __restrict__ grad, float* __restrict__ buf1,
                                                            float* __restrict__ x, float* __restrict__ row_sumsq,
                                                            int rows, int cols, float mu, const float* grad_scale) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float gs = grad_scale ? *grad_scale : 1.0f;
  const long long off = static_cast<long long>(row) * cols;
  float ss = 0.0f;
  for (int c = lane; c < cols; c += 32) {
    const float g = grad[off + c] * gs;
    const float b = buf1[off + c] + (1.0f - mu) * (g - buf1[off + c]);
    buf1[off + c] = b;
    const float xv = (1.0f - mu) * g + mu * b;
    x[off + c] = xv;
    ss += xv * xv;
  }
  ss = warp_sum(ss);
  if (lane == 0) row_sumsq[row] = ss;
}

__global__ void __launch_bounds__(256) muon_scale_rows_kernel(const float* __restrict__ x,
                                                              const float* __restrict__ row_scale,
                                                              const float* __restrict__ all_scale,
                                                              __nv_bfloat16* __restrict__ out, int rows, int cols) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float s = row_scale[row] * all_scale[0];
  const long long off = static_cast<long long>(row) * cols;
  for (int c = lane; c < cols; c += 32) out[off + c] = __float2bfloat16_rn(x[off + c] * s);
}

__global__ void __launch_bounds__(256) muon_apply_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ value,
                                                         const __nv_bfloat16* __restrict__ xb,
                                                         const float* __restrict__ scale0,
                                                         const float* __restrict__ line_scale, bool lines_are_rows,
                                                         int rows, int cols, float lr, float wd) {
  const long long n = static_cast<long long>(rows) * cols;
  const float s0 = scale0[0];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / cols), c = static_cast<int>(i - static_cast<long long>(r) * cols);
    const float x = __bfloat162float(xb[i]) * s0 * line_scale[lines_are_rows ? r : c];
    const float p = master[i];
    const float decay = (x * p >= 0.0f) ? lr * wd * p : 0.0f;
    const float pi = p - lr * x - decay;
    master[i] = pi;
    if (value != nullptr) value[i] = __float2bfloat16_rn(pi);
  }
}

// ---- batched forms: one launch per shape group (grid.y = matrix), 16-byte accesses --------------------------
// Stage 1 over P matrices given by pointer tables (gradients and momentum buffers live in different places).
__global__ void __launch_bounds__(256) muon_nesterov_batched_kernel(const long long* __restrict__ grad_ptrs,
                                                                    const long long* __restrict__ buf1_ptrs,
                                                                    float* __restrict__ x, float* __restrict__ row_sumsq,
                                                                    int rows, int cols, float mu,
                                                                    const float* grad_scale) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int p = blockIdx.y, lane = threadIdx.x & 31;
  const float gs = grad_scale ? *grad_scale : 1.0f;
  const long long off = static_cast<long long>(row) * cols;
  const float4* g4 = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grad_ptrs[p]) + off);
  float4* b4 = reinterpret_cast<float4*>(reinterpret_cast<float*>(buf1_ptrs[p]) + off);
  float4* x4 = reinterpret_cast<float4*>(x + (static_cast<long long>(p) * rows + row) * cols);
  float ss = 0.0f;
  for (int c = lane; c < cols / 4; c += 32) {
    const float4 g = g4[c];
    float4 b = b4[c];
    float4 xv;
    b.x += (1.0f - mu) * (g.x * gs - b.x), xv.x = (1.0f - mu) * g.x * gs + mu * b.x;
    b.y += (1.0f - mu) * (g.y * gs - b.y), xv.y = (1.0f - mu) * g.y * gs + mu * b.y;
    b.z += (1.0f - mu) * (g.z * gs - b.z), xv.z = (1.0f - mu) * g.z * gs + mu * b.z;
    b.w += (1.0f - mu) * (g.w * gs - b.w), xv.w = (1.0f - mu) * g.w * gs + mu * b.w;
    b4[c] = b;
    x4[c] = xv;
    ss += xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w;
  }
  ss = warp_sum(ss);
  if (lane == 0) row_sumsq[static_cast<long long>(p) * rows + row] = ss;
}

__global__ void __launch_bounds__(256) muon_scale_rows_batched_kernel(const float* __restrict__ x,
                                                                      const float* __restrict__ row_scale,
                                                                      const float* __restrict__ all_scale,
                                                                      __nv_bfloat16* __restrict__ out, int rows,
                                                                      int cols) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int p = blockIdx.y, lane = threadIdx.x & 31;
  const long long r = static_cast<long long>(p) * rows + row;
  const float s = row_scale[r] * all_scale[p];
  const float4* x4 = reinterpret_cast<const float4*>(x + r * cols);
  uint2* o2 = reinterpret_cast<uint2*>(out + r * cols);
  for (int c = lane; c < cols / 4; c += 32) {
    const float4 v = x4[c];
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * s, v.y * s), hi = __floats2bfloat162_rn(v.z * s, v.w * s);
    o2[c] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
  }
}

// Sum of squares along rows (reduce_cols: out[p, row]) or along columns (out[p, col]) of bf16 X [P, rows, cols].
__global__ void __launch_bounds__(256) muon_line_sumsq_kernel(const __nv_bfloat16* __restrict__ x,
                                                              float* __restrict__ out, int rows, int cols,
                                                              bool reduce_cols) {
  const int p = blockIdx.y;
  const __nv_bfloat16* xp = x + static_cast<long long>(p) * rows * cols;
  if (reduce_cols) {
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const uint4* r4 = reinterpret_cast<const uint4*>(xp + static_cast<long long>(row) * cols);
    float ss = 0.0f;
    for (int c = lane; c < cols / 8; c += 32) {
      const uint4 u = r4[c];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float a = __uint_as_float(w[e] << 16), b = __uint_as_float(w[e] & 0xffff0000u);
        ss += a * a + b * b;
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) out[static_cast<long long>(p) * rows + row] = ss;
  } else {
    // thread = pair of columns; rows are split over blockIdx.z-free loop (rows <= a few thousand)
    const int c2 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c2 >= cols / 2) return;
    float s0 = 0.0f, s1 = 0.0f;
    for (int r = 0; r < rows; ++r) {
      const uint32_t w = reinterpret_cast<const uint32_t*>(xp + static_cast<long long>(r) * cols)[c2];
      const float a = __uint_as_float(w << 16), b = __uint_as_float(w & 0xffff0000u);
      s0 += a * a, s1 += b * b;
    }
    out[static_cast<long long>(p) * cols + 2 * c2] = s0;
    out[static_cast<long long>(p) * cols + 2 * c2 + 1] = s1;
  }
}


// ---- the small per-matrix statistics of Muon, one CTA per matrix --------------------------------------------------
__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.0f;
#pragma unroll
  for (int w = 0; w < 8; ++w) t += red[w];
  return t;
}

// Row equilibration and Frobenius normalisation as one row scale (reference backends/cpu/kernels.cc:1667-1700):
//   row_scale[r] = (||X||_F / sqrt(rows)) / max(||row r||, 1e-6);  all_scale = 1 / (1.01 ||X diag(row_scale)||_F + 1e-6)
__global__ void __launch_bounds__(256) muon_prescale_kernel(const float* __restrict__ row_ss,
                                                            float* __restrict__ row_scale,
                                                            float* __restrict__ all_scale, int rows) {
  __shared__ float red[8];
  const int p = blockIdx.x;
  const float* ss = row_ss + static_cast<long long>(p) * rows;
  float* out = row_scale + static_cast<long long>(p) * rows;
  float t = 0.0f;
  for (int r = threadIdx.x; r < rows; r += 256) t += ss[r];
  const float frob = sqrtf(block_sum_256(t, red));
  const float target = frob / sqrtf(static_cast<float>(rows));
  float t2 = 0.0f;
  for (int r = threadIdx.x; r < rows; r += 256) {
    const float v = ss[r];
    const float sc = target / fmaxf(sqrtf(v), 1e-6f);
    out[r] = sc;
    t2 += v * sc * sc;
  }
  const float frob2 = sqrtf(block_sum_256(t2, red));
  if (threadIdx.x == 0) all_scale[p] = 1.0f / (frob2 * 1.01f + 1e-6f);
}

// Muon+ rescale, NorMuon second moment and per-line step (reference backends/cpu/kernels.cc:1746-1800):
//   scale = sqrt(min(rows, cols)) / max(||X||_F, 1e-6);  v = line_ss * scale^2 / line_len
//   buf2 += (1 - beta2)(v - buf2);  step = rsqrt(max(buf2, 1e-10))
//   line_scale = step * sqrt(sum v * line_len) / max(sqrt(sum v * line_len * step^2), 1e-10)
__global__ void __launch_bounds__(256) muon_poststats_kernel(const float* __restrict__ line_ss,
                                                             const long long* __restrict__ buf2_ptrs,
                                                             float* __restrict__ scale_out,
                                                             float* __restrict__ line_scale, int lines, int line_len,
                                                             float target_norm, float beta2) {
  __shared__ float red[8];
  const int p = blockIdx.x;
  const float* ss = line_ss + static_cast<long long>(p) * lines;
  float* buf2 = reinterpret_cast<float*>(buf2_ptrs[p]);
  float* out = line_scale + static_cast<long long>(p) * lines;
  float t = 0.0f;
  for (int i = threadIdx.x; i < lines; i += 256) t += ss[i];
  const float frob = sqrtf(block_sum_256(t, red));
  const float scale = target_norm / fmaxf(frob, 1e-6f);
  const float len = static_cast<float>(line_len);
  float tv = 0.0f, ts = 0.0f;
  for (int i = threadIdx.x; i < lines; i += 256) {
    const float v = ss[i] * (scale * scale) / len;
    float b = buf2[i];
    b += (1.0f - beta2) * (v - b);
    buf2[i] = b;
    const float step = rsqrtf(fmaxf(b, 1e-10f));
    out[i] = step;                       // finished below, once the two sums are known
    tv += v;
    ts += v * len * step * step;
  }
  const float v_norm = sqrtf(block_sum_256(tv, red) * len);
  const float denom = fmaxf(sqrtf(block_sum_256(ts, red)), 1e-10f);
  const float k = v_norm / denom;
  for (int i = threadIdx.x; i < lines; i += 256) out[i] *= k;
  if (threadIdx.x == 0) scale_out[p] = scale;
}

__global__ void __launch_bounds__(256) muon_apply_batched_kernel(const long long* __restrict__ master_ptrs,
                                                                 const long long* __restrict__ value_ptrs,
                                                                 const __nv_bfloat16* __restrict__ xb,
                                                                 const float* __restrict__ scale0,
                                                                 const float* __restrict__ line_scale,
                                                                 bool lines_are_rows, int rows, int cols, float lr,
                                                                 float wd) {
  const int p = blockIdx.y;
  float* master = reinterpret_cast<float*>(master_ptrs[p]);
  __nv_bfloat16* value = value_ptrs ? reinterpret_cast<__nv_bfloat16*>(value_ptrs[p]) : nullptr;
  const __nv_bfloat16* xp = xb + static_cast<long long>(p) * rows * cols;
  const int lines = lines_are_rows ? rows : cols;
  const float* ls = line_scale + static_cast<long long>(p) * lines;
  const float s0 = scale0[p];
  const long long n2 = static_cast<long long>(rows) * cols / 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n2;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i * 2;
    const int r = static_cast<int>(e / cols), c = static_cast<int>(e - static_cast<long long>(r) * cols);
    const uint32_t w = reinterpret_cast<const uint32_t*>(xp)[i];
    const float x0 = __uint_as_float(w << 16) * s0 * ls[lines_are_rows ? r : c];
    const float x1 = __uint_as_float(w & 0xffff0000u) * s0 * ls[lines_are_rows ? r : c + 1];
    float2 pm = reinterpret_cast<float2*>(master)[i];
    pm.x = pm.x - lr * x0 - ((x0 * pm.x >= 0.0f) ? lr * wd * pm.x : 0.0f);
    pm.y = pm.y - lr * x1 - ((x1 * pm.y >= 0.0f) ? lr * wd * pm.y : 0.0f);
    reinterpret_cast<float2*>(master)[i] = pm;
    if (value != nullptr) reinterpret_cast<__nv_bfloat162*>(value)[i] = __floats2bfloat162_rn(pm.x, pm.y);
  }
}

// The whole Muon step of a stack of small matrices (rows * cols <= 1024, e.g. the 10 x 12 value-gate projections and the
// 1 x 24 smear gate), one CTA per matrix, fp32 in shared memory: momentum and Nesterov blend, row equilibration and
// Frobenius normalisation, `ns_steps` Polar Express iterations, Muon+ rescale, NorMuon second moment and line step,
// cautious decay and update. Same arithmetic, in the same order, as the definition in ops/ref.py::muon_update
// (reference backends/cpu/kernels.cc:1614-1810); sums that the definition takes in double are taken in double here.
constexpr int kTinyMax = 1024;   // elements of one matrix
constexpr int kTinySide = 32;    // the smaller dimension

// Block-wide sum in a fixed order (every thread adds the same 128 partial sums): the result does not depend on how
// the warps are scheduled.
__device__ __forceinline__ double tiny_sum(double v, double* red) {
  __syncthreads();
  red[threadIdx.x] = v;
  __syncthreads();
  double t = 0.0;
  for (int w = 0; w < static_cast<int>(blockDim.x); ++w) t += red[w];
  return t;
}

struct TinyCoeffs {
  float c[5][3];
};

__global__ void __launch_bounds__(128) muon_tiny_kernel(const long long* __restrict__ grad_ptrs,
                                                        const long long* __restrict__ buf1_ptrs,
                                                        const long long* __restrict__ buf2_ptrs,
                                                        const long long* __restrict__ master_ptrs,
                                                        const long long* __restrict__ value_ptrs, int rows, int cols,
                                                        float mu, float beta2, float lr, float wd, int ns_steps,
                                                        const float* grad_scale, TinyCoeffs coeffs) {
  __shared__ float X[kTinyMax], Y[kTinyMax], A[kTinySide * kTinySide], Bm[kTinySide * kTinySide];
  __shared__ float line[kTinyMax];   // per-row scale, later per-line step (lines <= rows * cols)
  __shared__ double red[128];
  const int p = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
  const int n = rows * cols;
  const float* grad = reinterpret_cast<const float*>(grad_ptrs[p]);
  float* buf1 = reinterpret_cast<float*>(buf1_ptrs[p]);
  float* buf2 = reinterpret_cast<float*>(buf2_ptrs[p]);
  float* master = reinterpret_cast<float*>(master_ptrs[p]);
  __nv_bfloat16* value = value_ptrs != nullptr ? reinterpret_cast<__nv_bfloat16*>(value_ptrs[p]) : nullptr;
  const float gs = grad_scale ? *grad_scale : 1.0f;
  // 1. momentum, Nesterov blend
  double ss = 0.0;
  for (int i = tid; i < n; i += nt) {
    const float g = grad[i] * gs;
    const float b = buf1[i] + (1.0f - mu) * (g - buf1[i]);
    buf1[i] = b;
    const float x = (1.0f - mu) * g + mu * b;
    X[i] = x;
    ss += static_cast<double>(x) * x;
  }
  // 2. every row to the mean row norm
  const float frob = static_cast<float>(sqrt(tiny_sum(ss, red)));
  const float target = frob / sqrtf(static_cast<float>(rows));
  for (int r = tid; r < rows; r += nt) {
    double rs = 0.0;
    for (int c = 0; c < cols; ++c) rs += static_cast<double>(X[r * cols + c]) * X[r * cols + c];
    line[r] = target / fmaxf(static_cast<float>(sqrt(rs)), 1e-6f);
  }
  __syncthreads();
  ss = 0.0;
  for (int i = tid; i < n; i += nt) {
    const float x = X[i] * line[i / cols];
    X[i] = x;
    ss += static_cast<double>(x) * x;
  }
  // 3. Frobenius normalisation
  const float frob2 = static_cast<float>(sqrt(tiny_sum(ss, red)));
  const float inv_norm = 1.0f / (frob2 * 1.01f + 1e-6f);
  for (int i = tid; i < n; i += nt) X[i] *= inv_norm;
  __syncthreads();
  // 4. Polar Express: A = X^T X (tall) or X X^T, B = cb A + cc A A, X = ca X + X B (tall) or ca X + B X
  const bool tall = rows > cols;
  const int k = tall ? cols : rows;   // side of A
  float* Xc = X;
  float* Xn = Y;
  for (int it = 0; it < ns_steps && it < 5; ++it) {
    const float ca = coeffs.c[it][0], cb = coeffs.c[it][1], cc = coeffs.c[it][2];
    for (int e = tid; e < k * k; e += nt) {
      const int i = e / k, j = e - i * k;
      float acc = 0.0f;
      if (tall) {
        for (int r = 0; r < rows; ++r) acc += Xc[r * cols + i] * Xc[r * cols + j];
      } else {
        for (int c = 0; c < cols; ++c) acc += Xc[i * cols + c] * Xc[j * cols + c];
      }
      A[e] = acc;
    }
    __syncthreads();
    for (int e = tid; e < k * k; e += nt) {
      const int i = e / k, j = e - i * k;
      float acc = 0.0f;
      for (int q = 0; q < k; ++q) acc += A[i * k + q] * A[q * k + j];
      Bm[e] = cb * A[e] + cc * acc;
    }
    __syncthreads();
    for (int e = tid; e < n; e += nt) {
      const int r = e / cols, c = e - r * cols;
      float acc = 0.0f;
      if (tall) {
        for (int q = 0; q < cols; ++q) acc += Xc[r * cols + q] * Bm[q * k + c];
      } else {
        for (int q = 0; q < rows; ++q) acc += Bm[r * k + q] * Xc[q * cols + c];
      }
      Xn[e] = ca * Xc[e] + acc;
    }
    __syncthreads();
    float* t = Xc;
    Xc = Xn;
    Xn = t;
  }
  // 5. Muon+: snap the norm to sqrt(min(rows, cols))
  ss = 0.0;
  for (int i = tid; i < n; i += nt) ss += static_cast<double>(Xc[i]) * Xc[i];
  const float frob3 = static_cast<float>(sqrt(tiny_sum(ss, red)));
  const float snap = sqrtf(static_cast<float>(rows < cols ? rows : cols)) / fmaxf(frob3, 1e-6f);
  for (int i = tid; i < n; i += nt) Xc[i] *= snap;
  __syncthreads();
  // 6. NorMuon: second moment per line (rows when rows >= cols, else columns), normalised step
  const bool reduce_cols = rows >= cols;
  const int lines = reduce_cols ? rows : cols, line_len = reduce_cols ? cols : rows;
  double tv = 0.0, ts = 0.0;
  for (int l = tid; l < lines; l += nt) {
    double acc = 0.0;
    for (int q = 0; q < line_len; ++q) {
      const float x = reduce_cols ? Xc[l * cols + q] : Xc[q * cols + l];
      acc += static_cast<double>(x) * x;
    }
    const float v = static_cast<float>(acc / line_len);
    const float b = buf2[l] + (1.0f - beta2) * (v - buf2[l]);
    buf2[l] = b;
    const float step = 1.0f / sqrtf(fmaxf(b, 1e-10f));
    line[l] = step;
    tv += v;
    ts += static_cast<double>(v * static_cast<float>(line_len)) * step * step;
  }
  const float v_norm = sqrtf(static_cast<float>(tiny_sum(tv, red)) * static_cast<float>(line_len));
  const float denom = fmaxf(static_cast<float>(sqrt(tiny_sum(ts, red))), 1e-10f);
  const float kscale = v_norm / denom;
  // 7. cautious decay and update
  for (int i = tid; i < n; i += nt) {
    const int r = i / cols, c = i - r * cols;
    const float x = Xc[i] * (line[reduce_cols ? r : c] * kscale);
    const float pm = master[i];
    const float decay = (x * pm >= 0.0f) ? lr * wd * pm : 0.0f;
    const float q = pm - lr * x - decay;
    master[i] = q;
    if (value != nullptr) value[i] = __float2bfloat16_rn(q);
  }
}

__global__ void __launch_bounds__(256) relu2_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                    long long n) {
  const long long nv = n / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(x)[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float lo = fmaxf(__uint_as_float(w[e] << 16), 0.0f);
      const float hi = fmaxf(__uint_as_float(w[e] & 0xffff0000u), 0.0f);
      __nv_bfloat162 t = __floats2bfloat162_rn(lo * lo, hi * hi);
      o[e] = *reinterpret_cast<uint32_t*>(&t);
    }
    reinterpret_cast<uint4*>(y)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  if (blockIdx.x == 0) {
    for (long long i = nv * 8 + threadIdx.x; i < n; i += blockDim.x) {
      const float v = fmaxf(__bfloat162float(x[i]), 0.0f);
      y[i] = __float2bfloat16_rn(v * v);
    }
  }
}

__global__ void __launch_bounds__(256) cast_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                   long long n) {
  const long long nv = n / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
    __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 w;
    w.x = *reinterpret_cast<uint32_t*>(&lo);
    w.y = *reinterpret_cast<uint32_t*>(&hi);
    reinterpret_cast<uint2*>(y)[i] = w;
  }
  if (blockIdx.x == 0) {
    for (long long i = nv * 4 + threadIdx.x; i < n; i += blockDim.x) y[i] = __float2bfloat16_rn(x[i]);
  }
}

inline int grid_for(long long n, int per_thread) {
  long long b = (n / per_thread + 255) / 256;
  if (b < 1) b = 1;
  if (b > 148 * 16) b = 148 * 16;
  return static_cast<int>(b);
}

}  // namespace

#ifndef NC_EMU
void adamw_update(float* master, __nv_bfloat16* value, const float* grad, float* m, float* v, long long n, float lr,
                  float beta1, float beta2, float eps, float weight_decay, int step, const float* grad_scale,
                  cudaStream_t s) {
  if (n <= 0) return;
  const float bias1 = 1.0f - powf(beta1, static_cast<float>(step));
  const float bias2 = 1.0f - powf(beta2, static_cast<float>(step));
  adamw_kernel<<<grid_for(n, 4), 256, 0, s>>>(master, value, grad, m, v, n, lr, beta1, beta2, eps, weight_decay,
                                              1.0f / bias2, lr / bias1, grad_scale);
}
void muon_nesterov(const float* grad, float* buf1, float* x, float* row_sumsq, int rows, int cols, float momentum,
                   const float* grad_scale, cudaStream_t s) {
  if (rows <= 0) return;
  muon_nesterov_kernel<<<(rows + 7) / 8, 256, 0, s>>>(grad, buf1, x, row_sumsq, rows, cols, momentum, grad_scale);
}
void muon_scale_rows(const float* x, const float* row_scale, const float* all_scale, __nv_bfloat16* out, int rows,
                     int cols, cudaStream_t s) {
  if (rows <= 0) return;
  muon_scale_rows_kernel<<<(rows + 7) / 8, 256, 0, s>>>(x, row_scale, all_scale, out, rows, cols);
}
void muon_apply(float* master, __nv_bfloat16* value, const __nv_bfloat16* xb, const float* scale0,
                const float* line_scale, bool lines_are_rows, int rows, int cols, float lr, float weight_decay,
                cudaStream_t s) {
  const long long n = static_cast<long long>(rows) * cols;
  if (n <= 0) return;
  muon_apply_kernel<<<grid_for(n, 1), 256, 0, s>>>(master, value, xb, scale0, line_scale, lines_are_rows, rows, cols,
                                                   lr, weight_decay);
}
void relu2_bf16(const __nv_bfloat16* x, __nv_bfloat16* y, long long n, cudaStream_t s) {
  if (n <= 0) return;
  relu2_kernel<<<grid_for(n, 8), 256, 0, s>>>(x, y, n);
}
void cast_f32_bf16(const float* x, __nv_bfloat16* y, long long n, cudaStream_t s) {
  if (n <= 0) return;
  cast_kernel<<<grid_for(n, 4), 256, 0, s>>>(x, y, n);
}

const char* muon_tiny(const long long* grad_ptrs, const long long* buf1_ptrs, const long long* buf2_ptrs,
                      const long long* master_ptrs, const long long* value_ptrs, int P, int rows, int cols, float momentum,
                      float beta2, float lr, float weight_decay, int ns_steps, const float* grad_scale,
                      const double (*coeffs)[3], cudaStream_t s) {
  if (P <= 0) return nullptr;
  if (rows <= 0 || cols <= 0 || rows * cols > kTinyMax || (rows < cols ? rows : cols) > kTinySide)
    return "muon_tiny: at most 1024 elements per matrix and 32 on the smaller side";
  TinyCoeffs c;
  for (int i = 0; i < 5; ++i)
    for (int j = 0; j < 3; ++j) c.c[i][j] = static_cast<float>(coeffs[i][j]);
  muon_tiny_kernel<<<P, 128, 0, s>>>(grad_ptrs, buf1_ptrs, buf2_ptrs, master_ptrs, value_ptrs, rows, cols, momentum, beta2,
                                    lr, weight_decay, ns_steps, grad_scale, c);
  return nullptr;
}

void muon_nesterov_batched(const long long* grad_ptrs, const long long* buf1_ptrs, float* x, float* row_sumsq, int P,
                           int rows, int cols, float momentum, const float* grad_scale, cudaStream_t s) {
  if (P <= 0 || rows <= 0) return;
  muon_nesterov_batched_kernel<<<dim3((rows + 7) / 8, P), 256, 0, s>>>(grad_ptrs, buf1_ptrs, x, row_sumsq, rows, cols,
                                                                      momentum, grad_scale);
}
void muon_scale_rows_batched(const float* x, const float* row_scale, const float* all_scale, __nv_bfloat16* out, int P,
                             int rows, int cols, cudaStream_t s) {
  if (P <= 0 || rows <= 0) return;
  muon_scale_rows_batched_kernel<<<dim3((rows + 7) / 8, P), 256, 0, s>>>(x, row_scale, all_scale, out, rows, cols);
}
void muon_line_sumsq(const __nv_bfloat16* x, float* out, int P, int rows, int cols, bool reduce_cols, cudaStream_t s) {
  if (P <= 0 || rows <= 0) return;
  if (reduce_cols) {
    muon_line_sumsq_kernel<<<dim3((rows + 7) / 8, P), 256, 0, s>>>(x, out, rows, cols, true);
  } else {
    muon_line_sumsq_kernel<<<dim3((cols / 2 + 255) / 256, P), 256, 0, s>>>(x, out, rows, cols, false);
  }
}
void muon_prescale(const float* row_ss, float* row_scale, float* all_scale, int P, int rows, cudaStream_t s) {
  if (P > 0) muon_prescale_kernel<<<P, 256, 0, s>>>(row_ss, row_scale, all_scale, rows);
}
void muon_poststats(const float* line_ss, const long long* buf2_ptrs, float* scale_out, float* line_scale, int P,
                    int lines, int line_len, float target_norm, float beta2, cudaStream_t s) {
  if (P > 0)
    muon_poststats_kernel<<<P, 256, 0, s>>>(line_ss, buf2_ptrs, scale_out, line_scale, lines, line_len, target_norm,
                                            beta2);
}
void muon_apply_batched(const long long* master_ptrs, const long long* value_ptrs, const __nv_bfloat16* xb,
                        const float* scale0, const float* line_scale, bool lines_are_rows, int P, int rows, int cols,
                        float lr, float weight_decay, cudaStream_t s) {
  if (P <= 0 || rows <= 0) return;
  const long long n2 = static_cast<long long>(rows) * cols / 2;
  long long blocks = (n2 + 255) / 256;
  if (blocks > 296) blocks = 296;
  muon_apply_batched_kernel<<<dim3(static_cast<unsigned>(blocks), P), 256, 0, s>>>(
      master_ptrs, value_ptrs, xb, scale0, line_scale, lines_are_rows, rows, cols, lr, weight_decay);
}

#endif  // !NC_EMU

}  // namespace nc

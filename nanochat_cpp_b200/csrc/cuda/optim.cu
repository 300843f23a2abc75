// Optimizer kernels: fused AdamW, and the elementwise stages of Muon around its tensor-core products.
// The reference runs Muon as 39 launches per shape group with 17 small kernels
// (backends/cuda/kernels/muon.cu:83-464); here the momentum / Nesterov / row-norm stage, the row
// rescale + bf16 cast, and the NorMuon-scaled cautious update are one kernel each, and the Polar
// Express products run on the tcgen05 GEMM (batched over the matrices of a group).
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

}  // namespace nc

// Data-parallel communication kernels over NVLink peer memory (sm_100a).
//
// The reference synchronises gradients with a ring all-reduce staged through pinned host memory and TCP
// (backends/cuda/collective/native_sync.cu:130-194, ring_schedule.cc:93-160) and then runs a replicated
// optimizer. Here every parameter has one owner rank:
//   * `reduce_pull`  - the owner loads its segments of the gradient straight from every rank's buffer
//                      (plain peer loads through NVSwitch: one hop, no ring), sums in fixed rank order,
//                      scales, stores the result locally and accumulates the gradient-norm partial.
//   * `adamw_push` / `muon_apply_push` - the owner's update writes the new bf16 parameters into every
//                      rank's parameter buffer, so the parameter all-gather is the store of the update.
// Ordering across ranks uses flag words in symmetric memory: a rank publishes "bucket b of step s is
// final" after its backward kernels (stream order), the owner spins on the flags of all ranks before it
// loads. Every spin is bounded by a time budget and reports through the status word; nothing traps.
#include "comm.h"

#include <stdint.h>

#include "ptx.cuh"

namespace nc {

namespace {

__device__ bool wait_flags(const int* flags, int world, int slot, int value, int* status) {
  return wait_flags_bounded(flags + slot * world, world, value, status);
}

__global__ void signal_kernel(PeerPtrs flags, int world, int my_rank, int slot, int value) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    st_release_sys(static_cast<int*>(flags.p[r]) + slot * world + my_rank, value);
  }
}

__global__ void wait_kernel(const int* flags, int world, int slot, int value, int* status,
                            unsigned long long budget_ns) {
  if (threadIdx.x == 0) wait_flags_bounded(flags + slot * world, world, value, status, budget_ns);
}

constexpr int kReduceUnroll = 4;
constexpr int kRankGroup = 4;
constexpr int kMaxSegs = 64;

__global__ void __launch_bounds__(256) reduce_pull_kernel(PeerPtrs grads, int world, int my_rank,
                                                          const Segment* __restrict__ segs, int nsegs,
                                                          long long total, float scale, const int* flags, int slot,
                                                          int value, double* sumsq, int* status) {
  __shared__ int ok_sh;
  __shared__ double red[8];
  __shared__ long long seg_first[kMaxSegs + 1];  // first vector index of every segment in the concatenated space
  __shared__ long long seg_off[kMaxSegs];
  if (threadIdx.x == 0) {
    ok_sh = wait_flags(flags, world, slot, value, status) ? 1 : 0;
    long long acc = 0;
    for (int i = 0; i < nsegs; ++i) {
      seg_first[i] = acc;
      seg_off[i] = segs[i].offset;
      acc += segs[i].count / 4;
    }
    seg_first[nsegs] = acc;
  }
  __syncthreads();
  if (!ok_sh) return;
  double acc = 0.0;
  float acc_f = 0.0f;   // squares are added in fp32 and folded into the fp64 sum once per loop trip (16 terms)
  const long long nvec = total / 4;
  const long long threads = static_cast<long long>(gridDim.x) * blockDim.x;
  float* mine = static_cast<float*>(grads.p[my_rank]);
  // kReduceUnroll independent 16-byte peer loads per rank are in flight per thread: NVLink latency is hidden by
  // memory-level parallelism, not by occupancy
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < nvec;
       i0 += threads * kReduceUnroll) {
    long long e[kReduceUnroll];
    float4 sum[kReduceUnroll];
#pragma unroll
    for (int u = 0; u < kReduceUnroll; ++u) {
      const long long i = i0 + u * threads;
      e[u] = -1;
      sum[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < nvec) {
        int lo = 0, hi = nsegs - 1;
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (seg_first[mid] <= i) lo = mid; else hi = mid - 1;
        }
        e[u] = seg_off[lo] + (i - seg_first[lo]) * 4;
      }
    }
    // ranks are read kRankGroup at a time: kRankGroup * kReduceUnroll loads are issued before the first one is
    // consumed, so a trip over 8 ranks pays two NVLink round trips instead of eight. The sum order (rank 0, 1, ...)
    // is the same on every owner.
    for (int r0 = 0; r0 < world; r0 += kRankGroup) {
      float4 v[kRankGroup][kReduceUnroll];
#pragma unroll
      for (int g = 0; g < kRankGroup; ++g) {
        const float* src = static_cast<const float*>(grads.p[min(r0 + g, world - 1)]);
        const bool live = r0 + g < world;
#pragma unroll
        for (int u = 0; u < kReduceUnroll; ++u)
          v[g][u] = (live && e[u] >= 0) ? *reinterpret_cast<const float4*>(src + e[u]) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int g = 0; g < kRankGroup; ++g) {
#pragma unroll
        for (int u = 0; u < kReduceUnroll; ++u) {
          sum[u].x += v[g][u].x, sum[u].y += v[g][u].y, sum[u].z += v[g][u].z, sum[u].w += v[g][u].w;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kReduceUnroll; ++u) {
      if (e[u] < 0) continue;
      float4 q = sum[u];
      q.x *= scale, q.y *= scale, q.z *= scale, q.w *= scale;
      *reinterpret_cast<float4*>(mine + e[u]) = q;
      acc_f += q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
    }
    acc += static_cast<double>(acc_f);
    acc_f = 0.0f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < 8; ++w) t += red[w];
    atomicAdd(sumsq, t);
  }
}

__global__ void __launch_bounds__(256) adamw_push_kernel(float* __restrict__ master, PeerPtrs values,
                                                         long long value_offset, int world,
                                                         const float* __restrict__ grad, float* __restrict__ m,
                                                         float* __restrict__ v, long long n, float lr, float beta1,
                                                         float beta2, float eps, float wd, float inv_bias2,
                                                         float step_size, const float* grad_scale) {
  const float gs = grad_scale ? *grad_scale : 1.0f;
  const float decay = 1.0f - lr * wd;
  const long long nv = n / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 p4 = reinterpret_cast<float4*>(master)[i];
    const float4 g4 = reinterpret_cast<const float4*>(grad)[i];
    const float4 m4 = reinterpret_cast<float4*>(m)[i];
    const float4 v4 = reinterpret_cast<float4*>(v)[i];
    float pp[4] = {p4.x, p4.y, p4.z, p4.w};
    const float gg[4] = {g4.x, g4.y, g4.z, g4.w};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float g = gg[e] * gs;
      float pi = pp[e] * decay;
      mm[e] = mm[e] + (1.0f - beta1) * (g - mm[e]);
      vv[e] = vv[e] + (1.0f - beta2) * (g * g - vv[e]);
      pi -= step_size * (mm[e] / (sqrtf(vv[e] * inv_bias2) + eps));
      pp[e] = pi;
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]);
    __nv_bfloat162 hi = __floats2bfloat162_rn(pp[2], pp[3]);
    uint2 w;
    w.x = *reinterpret_cast<uint32_t*>(&lo);
    w.y = *reinterpret_cast<uint32_t*>(&hi);
    for (int r = 0; r < world; ++r)
      reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(values.p[r]) + value_offset)[i] = w;
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
      for (int r = 0; r < world; ++r) (static_cast<__nv_bfloat16*>(values.p[r]) + value_offset)[i] = __float2bfloat16_rn(pi);
    }
  }
}

__global__ void __launch_bounds__(256) muon_apply_push_kernel(float* __restrict__ master, PeerPtrs values,
                                                              long long value_offset, int world,
                                                              const __nv_bfloat16* __restrict__ xb,
                                                              const float* __restrict__ scale0,
                                                              const float* __restrict__ line_scale,
                                                              bool lines_are_rows, int rows, int cols, float lr,
                                                              float wd) {
  const long long n2 = static_cast<long long>(rows) * cols / 2;  // cols is even
  const float s0 = scale0[0];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n2;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i * 2;
    const int r = static_cast<int>(e / cols), c = static_cast<int>(e - static_cast<long long>(r) * cols);
    const __nv_bfloat162 xv = reinterpret_cast<const __nv_bfloat162*>(xb)[i];
    const float2 p = reinterpret_cast<const float2*>(master)[i];
    const float ls0 = line_scale[lines_are_rows ? r : c];
    const float ls1 = line_scale[lines_are_rows ? r : c + 1];
    const float x0 = __bfloat162float(xv.x) * s0 * ls0;
    const float x1 = __bfloat162float(xv.y) * s0 * ls1;
    const float q0 = p.x - lr * x0 - ((x0 * p.x >= 0.0f) ? lr * wd * p.x : 0.0f);
    const float q1 = p.y - lr * x1 - ((x1 * p.y >= 0.0f) ? lr * wd * p.y : 0.0f);
    reinterpret_cast<float2*>(master)[i] = make_float2(q0, q1);
    const __nv_bfloat162 o = __floats2bfloat162_rn(q0, q1);
    for (int k = 0; k < world; ++k)
      reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(values.p[k]) + value_offset)[i] = o;
  }
}

inline int grid_for(long long n, int per_thread, int cap) {
  long long b = (n / per_thread + 255) / 256;
  if (b < 1) b = 1;
  if (b > cap) b = cap;
  return static_cast<int>(b);
}

}  // namespace

void comm_signal(const PeerPtrs& flags, int world, int my_rank, int slot, int value, cudaStream_t s) {
  signal_kernel<<<1, 32, 0, s>>>(flags, world, my_rank, slot, value);
}
void comm_wait(const int* local_flags, int world, int slot, int value, int* status, cudaStream_t s, int budget_ms) {
  const unsigned long long budget = budget_ms > 0 ? static_cast<unsigned long long>(budget_ms) * 1000000ull
                                                  : kPeerWaitBudgetNs;
  wait_kernel<<<1, 32, 0, s>>>(local_flags, world, slot, value, status, budget);
}
void comm_reduce_pull(const PeerPtrs& grads, int world, int my_rank, const Segment* segs_dev, int nsegs,
                      long long total, float scale, const int* local_flags, int slot, int value, double* sumsq,
                      int* status, int ctas, cudaStream_t s) {
  if (total <= 0 || nsegs <= 0 || nsegs > kMaxSegs) return;
  reduce_pull_kernel<<<ctas, 256, 0, s>>>(grads, world, my_rank, segs_dev, nsegs, total, scale, local_flags, slot,
                                          value, sumsq, status);
}
void comm_adamw_push(float* master, const PeerPtrs& values, long long value_offset, int world, const float* grad,
                     float* m, float* v, long long n, float lr, float beta1, float beta2, float eps,
                     float weight_decay, int step, const float* grad_scale, cudaStream_t s) {
  if (n <= 0) return;
  const float bias1 = 1.0f - powf(beta1, static_cast<float>(step));
  const float bias2 = 1.0f - powf(beta2, static_cast<float>(step));
  adamw_push_kernel<<<grid_for(n, 4, 148 * 8), 256, 0, s>>>(master, values, value_offset, world, grad, m, v, n, lr,
                                                           beta1, beta2, eps, weight_decay, 1.0f / bias2, lr / bias1,
                                                           grad_scale);
}
void comm_muon_apply_push(float* master, const PeerPtrs& values, long long value_offset, int world,
                          const __nv_bfloat16* xb, const float* scale0, const float* line_scale,
                          bool lines_are_rows, int rows, int cols, float lr, float weight_decay, cudaStream_t s) {
  const long long n = static_cast<long long>(rows) * cols;
  if (n <= 0) return;
  muon_apply_push_kernel<<<grid_for(n, 2, 148 * 8), 256, 0, s>>>(master, values, value_offset, world, xb, scale0,
                                                                line_scale, lines_are_rows, rows, cols, lr,
                                                                weight_decay);
}

}  // namespace nc

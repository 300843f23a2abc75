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
#include "host_build.h"

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


// ---------------------------------------------------------------------------------------------------------
// Reduce-scatter with bf16 on the wire, by stores.
//
// `grad_push`: when a bucket of this rank's fp32 gradient is final, every element that another rank owns is
// scaled, rounded to bf16 and stored straight into that owner's receive buffer (slot [my_rank]) over NVLink:
// posted 16-byte stores, no round trip, half the bytes of the fp32 pull. `grad_reduce_local`: the owner waits
// (bounded) for the bucket's flag of every rank, then sums, for each element it owns, its own fp32 value and the
// N-1 bf16 values it received, in fixed rank order, in fp32; the result replaces its local gradient and its
// square goes into the gradient-norm partial. Everything the reduction reads is local HBM.
// ---------------------------------------------------------------------------------------------------------
constexpr int kMaxPushSegs = 128;
constexpr int kPushUnroll = 4;

struct PushSeg {       // one contiguous run of elements owned by `dst_rank`
  long long first_vec;  // index of its first 8-element vector in the launch's concatenated space
  long long src_off;    // element offset in the flat gradient buffer
  long long dst_pos;    // element position in the owner's receive slot (multiple of 8)
  long long dst_rank;
  long long count;      // elements
};

__device__ __forceinline__ int find_seg(const long long* first, int nsegs, long long i) {
  int lo = 0, hi = nsegs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (first[mid] <= i) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(256) grad_push_kernel(const float* __restrict__ grad, PeerPtrs recv,
                                                        long long recv_stride, int my_rank,
                                                        const PushSeg* __restrict__ segs, int nsegs, long long nvec,
                                                        float scale) {
  __shared__ long long s_first[kMaxPushSegs];
  __shared__ long long s_src[kMaxPushSegs], s_dst[kMaxPushSegs], s_cnt[kMaxPushSegs];
  __shared__ int s_rank[kMaxPushSegs];
  for (int i = threadIdx.x; i < nsegs; i += blockDim.x) {
    s_first[i] = segs[i].first_vec, s_src[i] = segs[i].src_off, s_dst[i] = segs[i].dst_pos;
    s_cnt[i] = segs[i].count, s_rank[i] = static_cast<int>(segs[i].dst_rank);
  }
  __syncthreads();
  const long long threads = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < nvec;
       i0 += threads * kPushUnroll) {
    float4 a[kPushUnroll], b[kPushUnroll];
    __nv_bfloat16* dst[kPushUnroll];
    int full[kPushUnroll];
#pragma unroll
    for (int u = 0; u < kPushUnroll; ++u) {
      const long long i = i0 + u * threads;
      dst[u] = nullptr, full[u] = 0;
      if (i >= nvec) continue;
      const int sg = find_seg(s_first, nsegs, i);
      const long long k = (i - s_first[sg]) * 8;
      const long long left = s_cnt[sg] - k;
      const float* src = grad + s_src[sg] + k;
      dst[u] = static_cast<__nv_bfloat16*>(recv.p[s_rank[sg]]) + my_rank * recv_stride + s_dst[sg] + k;
      if (left >= 8) {
        full[u] = 1;
        a[u] = *reinterpret_cast<const float4*>(src);
        b[u] = *reinterpret_cast<const float4*>(src + 4);
      } else {
        for (int e = 0; e < static_cast<int>(left); ++e) dst[u][e] = __float2bfloat16_rn(src[e] * scale);
        dst[u] = nullptr;
      }
    }
#pragma unroll
    for (int u = 0; u < kPushUnroll; ++u) {
      if (dst[u] == nullptr || !full[u]) continue;
      uint4 w;
      w.x = pack_bf16x2(a[u].x * scale, a[u].y * scale);
      w.y = pack_bf16x2(a[u].z * scale, a[u].w * scale);
      w.z = pack_bf16x2(b[u].x * scale, b[u].y * scale);
      w.w = pack_bf16x2(b[u].z * scale, b[u].w * scale);
      *reinterpret_cast<uint4*>(dst[u]) = w;
    }
  }
}

struct OwnSeg {
  long long first_vec;
  long long off;    // element offset in the flat gradient buffer
  long long pos;    // element position in the receive slots (multiple of 8)
  long long count;  // elements
};

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& w) {
  const uint32_t v[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    acc[2 * j] += __uint_as_float(v[j] << 16);
    acc[2 * j + 1] += __uint_as_float(v[j] & 0xffff0000u);
  }
}

__global__ void __launch_bounds__(256) grad_reduce_local_kernel(float* __restrict__ grad,
                                                                const __nv_bfloat16* __restrict__ recv,
                                                                long long recv_stride, int world, int my_rank,
                                                                const OwnSeg* __restrict__ segs, int nsegs,
                                                                long long nvec, float scale, const int* flags,
                                                                int slot, int value, double* sumsq, int* status) {
  __shared__ int ok_sh;
  __shared__ double red[8];
  __shared__ long long s_first[kMaxSegs], s_off[kMaxSegs], s_pos[kMaxSegs], s_cnt[kMaxSegs];
  if (threadIdx.x == 0) ok_sh = wait_flags(flags, world, slot, value, status) ? 1 : 0;
  for (int i = threadIdx.x; i < nsegs; i += blockDim.x) {
    s_first[i] = segs[i].first_vec, s_off[i] = segs[i].off, s_pos[i] = segs[i].pos, s_cnt[i] = segs[i].count;
  }
  __syncthreads();
  if (!ok_sh) return;
  double acc = 0.0;
  const long long threads = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += threads) {
    const int sg = find_seg(s_first, nsegs, i);
    const long long k = (i - s_first[sg]) * 8;
    const long long left = s_cnt[sg] - k;
    float* mine = grad + s_off[sg] + k;
    const __nv_bfloat16* slot0 = recv + s_pos[sg] + k;
    float sum[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) sum[e] = 0.0f;
    if (left >= 8) {
      uint4 w[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < world && r != my_rank) w[r] = *reinterpret_cast<const uint4*>(slot0 + r * recv_stride);
      const float4 a = *reinterpret_cast<const float4*>(mine), b = *reinterpret_cast<const float4*>(mine + 4);
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {     // fixed rank order: the same sum on every run
        if (r >= world) continue;
        if (r == my_rank) {
          sum[0] += a.x * scale, sum[1] += a.y * scale, sum[2] += a.z * scale, sum[3] += a.w * scale;
          sum[4] += b.x * scale, sum[5] += b.y * scale, sum[6] += b.z * scale, sum[7] += b.w * scale;
        } else {
          add_bf16x8(sum, w[r]);
        }
      }
      *reinterpret_cast<float4*>(mine) = make_float4(sum[0], sum[1], sum[2], sum[3]);
      *reinterpret_cast<float4*>(mine + 4) = make_float4(sum[4], sum[5], sum[6], sum[7]);
      float sq = 0.0f;
#pragma unroll
      for (int e = 0; e < 8; ++e) sq = fmaf(sum[e], sum[e], sq);
      acc += static_cast<double>(sq);
    } else {
      for (int e = 0; e < static_cast<int>(left); ++e) {
        float t = 0.0f;
        for (int r = 0; r < world; ++r)
          t += r == my_rank ? mine[e] * scale : __bfloat162float(slot0[r * recv_stride + e]);
        mine[e] = t;
        acc += static_cast<double>(t) * t;
      }
    }
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

// Eight parameters per thread: the bf16 results leave as ONE 16-byte store per destination rank. NVLink carries
// stores as packets with a fixed header, so 16-byte stores move about twice the payload per packet of the 8-byte
// stores a four-wide kernel would issue.
// Stores of an owner's new bf16 parameters into every rank's buffer: one plain store per rank through its peer
// pointer, or, when the buffer has an NVLink multicast address (values.mc), ONE multimem.st: the switch replicates it
// to every rank, this one included, so the bytes on this GPU's links drop from (world - 1) x to 1 x. The flag that
// publishes the data is a release store issued by a later kernel on the same stream, as for the plain stores.
// (multimem.st has no 2-byte form: single odd elements always go through the peer pointers.)
__device__ __forceinline__ void store_all16(const PeerPtrs& values, int world, long long elem, const uint4& w) {
#ifndef NC_EMU
  if (values.mc != nullptr) {
    __nv_bfloat16* a = static_cast<__nv_bfloat16*>(values.mc) + elem;
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(a), "r"(w.x), "r"(w.y), "r"(w.z),
                 "r"(w.w)
                 : "memory");
    return;
  }
#endif
  for (int k = 0; k < world; ++k) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(values.p[k]) + elem) = w;
}
__device__ __forceinline__ void store_all4(const PeerPtrs& values, int world, long long elem, uint32_t w) {
#ifndef NC_EMU
  if (values.mc != nullptr) {
    __nv_bfloat16* a = static_cast<__nv_bfloat16*>(values.mc) + elem;
    asm volatile("multimem.st.relaxed.sys.global.bf16x2 [%0], %1;" ::"l"(a), "r"(w) : "memory");
    return;
  }
#endif
  for (int k = 0; k < world; ++k) *reinterpret_cast<uint32_t*>(static_cast<__nv_bfloat16*>(values.p[k]) + elem) = w;
}
__device__ __forceinline__ void store_all2(const PeerPtrs& values, int world, long long elem, __nv_bfloat16 h) {
  for (int k = 0; k < world; ++k) (static_cast<__nv_bfloat16*>(values.p[k]) + elem)[0] = h;
}

__global__ void __launch_bounds__(256) adamw_push_kernel(float* __restrict__ master, PeerPtrs values,
                                                         long long value_offset, int world,
                                                         const float* __restrict__ grad, float* __restrict__ m,
                                                         float* __restrict__ v, long long n, float lr, float beta1,
                                                         float beta2, float eps, float wd, float inv_bias2,
                                                         float step_size, const float* grad_scale) {
  const float gs = grad_scale ? *grad_scale : 1.0f;
  const float decay = 1.0f - lr * wd;
  const long long nv = n / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float pp[8], gg[8], mm[8], vv[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 p4 = reinterpret_cast<const float4*>(master)[2 * i + h];
      const float4 g4 = reinterpret_cast<const float4*>(grad)[2 * i + h];
      const float4 m4 = reinterpret_cast<const float4*>(m)[2 * i + h];
      const float4 v4 = reinterpret_cast<const float4*>(v)[2 * i + h];
      pp[4 * h] = p4.x, pp[4 * h + 1] = p4.y, pp[4 * h + 2] = p4.z, pp[4 * h + 3] = p4.w;
      gg[4 * h] = g4.x, gg[4 * h + 1] = g4.y, gg[4 * h + 2] = g4.z, gg[4 * h + 3] = g4.w;
      mm[4 * h] = m4.x, mm[4 * h + 1] = m4.y, mm[4 * h + 2] = m4.z, mm[4 * h + 3] = m4.w;
      vv[4 * h] = v4.x, vv[4 * h + 1] = v4.y, vv[4 * h + 2] = v4.z, vv[4 * h + 3] = v4.w;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float g = gg[e] * gs;
      float pi = pp[e] * decay;
      mm[e] = mm[e] + (1.0f - beta1) * (g - mm[e]);
      vv[e] = vv[e] + (1.0f - beta2) * (g * g - vv[e]);
      pi -= step_size * (mm[e] / (sqrtf(vv[e] * inv_bias2) + eps));
      pp[e] = pi;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      reinterpret_cast<float4*>(master)[2 * i + h] = make_float4(pp[4 * h], pp[4 * h + 1], pp[4 * h + 2], pp[4 * h + 3]);
      reinterpret_cast<float4*>(m)[2 * i + h] = make_float4(mm[4 * h], mm[4 * h + 1], mm[4 * h + 2], mm[4 * h + 3]);
      reinterpret_cast<float4*>(v)[2 * i + h] = make_float4(vv[4 * h], vv[4 * h + 1], vv[4 * h + 2], vv[4 * h + 3]);
    }
    uint4 w;
    w.x = pack_bf16x2(pp[0], pp[1]), w.y = pack_bf16x2(pp[2], pp[3]);
    w.z = pack_bf16x2(pp[4], pp[5]), w.w = pack_bf16x2(pp[6], pp[7]);
    store_all16(values, world, value_offset + i * 8, w);
  }
  if (blockIdx.x == 0) {
    for (long long i = nv * 8 + threadIdx.x; i < n; i += blockDim.x) {
      const float g = grad[i] * gs;
      float pi = master[i] * decay;
      const float mi = m[i] + (1.0f - beta1) * (g - m[i]);
      const float vi = v[i] + (1.0f - beta2) * (g * g - v[i]);
      m[i] = mi;
      v[i] = vi;
      pi -= step_size * (mi / (sqrtf(vi * inv_bias2) + eps));
      master[i] = pi;
      store_all2(values, world, value_offset + i, __float2bfloat16_rn(pi));
    }
  }
}

// VEC = 8 when cols is a multiple of 8 (one 16-byte store per destination rank), else 2.
template <int VEC>
__global__ void __launch_bounds__(256) muon_apply_push_kernel(float* __restrict__ master, PeerPtrs values,
                                                              long long value_offset, int world,
                                                              const __nv_bfloat16* __restrict__ xb,
                                                              const float* __restrict__ scale0,
                                                              const float* __restrict__ line_scale,
                                                              bool lines_are_rows, int rows, int cols, float lr,
                                                              float wd) {
  const long long nv = static_cast<long long>(rows) * cols / VEC;  // cols is a multiple of VEC
  const float s0 = scale0[0];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e0 = i * VEC;
    const int r = static_cast<int>(e0 / cols), c = static_cast<int>(e0 - static_cast<long long>(r) * cols);
    float x[VEC], p[VEC];
    if constexpr (VEC == 8) {
      const uint4 xw = reinterpret_cast<const uint4*>(xb)[i];
      const uint32_t xv[4] = {xw.x, xw.y, xw.z, xw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) x[2 * j] = __uint_as_float(xv[j] << 16), x[2 * j + 1] = __uint_as_float(xv[j] & 0xffff0000u);
      const float4 pa = reinterpret_cast<const float4*>(master)[2 * i], pb = reinterpret_cast<const float4*>(master)[2 * i + 1];
      p[0] = pa.x, p[1] = pa.y, p[2] = pa.z, p[3] = pa.w, p[4] = pb.x, p[5] = pb.y, p[6] = pb.z, p[7] = pb.w;
    } else {
      const __nv_bfloat162 xv = reinterpret_cast<const __nv_bfloat162*>(xb)[i];
      x[0] = __bfloat162float(xv.x), x[1] = __bfloat162float(xv.y);
      const float2 pv = reinterpret_cast<const float2*>(master)[i];
      p[0] = pv.x, p[1] = pv.y;
    }
    const float row_ls = lines_are_rows ? line_scale[r] : 0.0f;
    float q[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float ls = lines_are_rows ? row_ls : line_scale[c + j];
      const float xx = x[j] * s0 * ls;
      q[j] = p[j] - lr * xx - ((xx * p[j] >= 0.0f) ? lr * wd * p[j] : 0.0f);
    }
    if constexpr (VEC == 8) {
      reinterpret_cast<float4*>(master)[2 * i] = make_float4(q[0], q[1], q[2], q[3]);
      reinterpret_cast<float4*>(master)[2 * i + 1] = make_float4(q[4], q[5], q[6], q[7]);
      uint4 w;
      w.x = pack_bf16x2(q[0], q[1]), w.y = pack_bf16x2(q[2], q[3]), w.z = pack_bf16x2(q[4], q[5]), w.w = pack_bf16x2(q[6], q[7]);
      store_all16(values, world, value_offset + i * 8, w);
    } else {
      reinterpret_cast<float2*>(master)[i] = make_float2(q[0], q[1]);
      const uint32_t w = pack_bf16x2(q[0], q[1]);
      store_all4(values, world, value_offset + i * 2, w);
    }
  }
}

// The same update for a whole shape group in one launch: blockIdx.y selects the matrix; `master_ptrs[p]` is its
// fp32 master and `value_offsets[p]` its element offset in every rank's parameter buffer. cols % 8 == 0.
__global__ void __launch_bounds__(256) muon_apply_push_batched_kernel(const long long* __restrict__ master_ptrs,
                                                                      const long long* __restrict__ value_offsets,
                                                                      PeerPtrs values, int world,
                                                                      const __nv_bfloat16* __restrict__ xb,
                                                                      const float* __restrict__ scale0,
                                                                      const float* __restrict__ line_scale,
                                                                      bool lines_are_rows, int rows, int cols, float lr,
                                                                      float wd) {
  const int p = blockIdx.y;
  float* master = reinterpret_cast<float*>(master_ptrs[p]);
  const long long value_offset = value_offsets[p];
  const __nv_bfloat16* xp = xb + static_cast<long long>(p) * rows * cols;
  const float* lsp = line_scale + static_cast<long long>(p) * (lines_are_rows ? rows : cols);
  const float s0 = scale0[p];
  const long long nv = static_cast<long long>(rows) * cols / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e0 = i * 8;
    const int r = static_cast<int>(e0 / cols), c = static_cast<int>(e0 - static_cast<long long>(r) * cols);
    const uint4 xw = reinterpret_cast<const uint4*>(xp)[i];
    const uint32_t xv[4] = {xw.x, xw.y, xw.z, xw.w};
    const float4 pa = reinterpret_cast<const float4*>(master)[2 * i], pb = reinterpret_cast<const float4*>(master)[2 * i + 1];
    const float pm[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
    const float row_ls = lines_are_rows ? lsp[r] : 0.0f;
    float q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float xraw = (j & 1) ? __uint_as_float(xv[j >> 1] & 0xffff0000u) : __uint_as_float(xv[j >> 1] << 16);
      const float xx = xraw * s0 * (lines_are_rows ? row_ls : lsp[c + j]);
      q[j] = pm[j] - lr * xx - ((xx * pm[j] >= 0.0f) ? lr * wd * pm[j] : 0.0f);
    }
    reinterpret_cast<float4*>(master)[2 * i] = make_float4(q[0], q[1], q[2], q[3]);
    reinterpret_cast<float4*>(master)[2 * i + 1] = make_float4(q[4], q[5], q[6], q[7]);
    uint4 w;
    w.x = pack_bf16x2(q[0], q[1]), w.y = pack_bf16x2(q[2], q[3]), w.z = pack_bf16x2(q[4], q[5]), w.w = pack_bf16x2(q[6], q[7]);
    store_all16(values, world, value_offset + i * 8, w);
  }
}

inline int grid_for(long long n, int per_thread, int cap) {
  long long b = (n / per_thread + 255) / 256;
  if (b < 1) b = 1;
  if (b > cap) b = cap;
  return static_cast<int>(b);
}

}  // namespace

#ifndef NC_EMU
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
void comm_grad_push(const float* grad, const PeerPtrs& recv, long long recv_stride, int my_rank,
                    const long long* segs_dev, int nsegs, long long nvec, float scale, int ctas, cudaStream_t s) {
  if (nvec <= 0 || nsegs <= 0 || nsegs > kMaxPushSegs) return;
  static_assert(sizeof(PushSeg) == 5 * sizeof(long long), "PushSeg layout");
  long long want = (nvec + 256 * kPushUnroll - 1) / (256 * kPushUnroll);
  if (want < ctas) ctas = static_cast<int>(want < 1 ? 1 : want);
  grad_push_kernel<<<ctas, 256, 0, s>>>(grad, recv, recv_stride, my_rank, reinterpret_cast<const PushSeg*>(segs_dev),
                                        nsegs, nvec, scale);
}
void comm_grad_reduce_local(float* grad, const __nv_bfloat16* recv, long long recv_stride, int world, int my_rank,
                            const long long* segs_dev, int nsegs, long long nvec, float scale,
                            const int* local_flags, int slot, int value, double* sumsq, int* status, int ctas,
                            cudaStream_t s) {
  if (nvec <= 0 || nsegs <= 0 || nsegs > kMaxSegs) return;
  static_assert(sizeof(OwnSeg) == 4 * sizeof(long long), "OwnSeg layout");
  long long want = (nvec + 255) / 256;
  if (want < ctas) ctas = static_cast<int>(want < 1 ? 1 : want);
  grad_reduce_local_kernel<<<ctas, 256, 0, s>>>(grad, recv, recv_stride, world, my_rank,
                                                reinterpret_cast<const OwnSeg*>(segs_dev), nsegs, nvec, scale,
                                                local_flags, slot, value, sumsq, status);
}
void comm_adamw_push(float* master, const PeerPtrs& values, long long value_offset, int world, const float* grad,
                     float* m, float* v, long long n, float lr, float beta1, float beta2, float eps,
                     float weight_decay, int step, const float* grad_scale, cudaStream_t s, int max_ctas) {
  if (n <= 0) return;
  const float bias1 = 1.0f - powf(beta1, static_cast<float>(step));
  const float bias2 = 1.0f - powf(beta2, static_cast<float>(step));
  // max_ctas: eight CTAs of 256 threads fill every thread slot of an SM; beside the Newton-Schulz products (one
  // 200 KB CTA per SM) the caller asks for two, so that those CTAs can become resident at once
  adamw_push_kernel<<<grid_for(n, 8, max_ctas > 0 ? max_ctas : 148 * 8), 256, 0, s>>>(master, values, value_offset, world, grad, m, v, n, lr,
                                                           beta1, beta2, eps, weight_decay, 1.0f / bias2, lr / bias1,
                                                           grad_scale);
}
void comm_muon_apply_push(float* master, const PeerPtrs& values, long long value_offset, int world,
                          const __nv_bfloat16* xb, const float* scale0, const float* line_scale,
                          bool lines_are_rows, int rows, int cols, float lr, float weight_decay, cudaStream_t s) {
  const long long n = static_cast<long long>(rows) * cols;
  if (n <= 0) return;
  if (cols % 8 == 0 && value_offset % 8 == 0)
    muon_apply_push_kernel<8><<<grid_for(n, 8, 148 * 8), 256, 0, s>>>(master, values, value_offset, world, xb, scale0,
                                                                     line_scale, lines_are_rows, rows, cols, lr,
                                                                     weight_decay);
  else
    muon_apply_push_kernel<2><<<grid_for(n, 2, 148 * 8), 256, 0, s>>>(master, values, value_offset, world, xb, scale0,
                                                                     line_scale, lines_are_rows, rows, cols, lr,
                                                                     weight_decay);
}

void comm_muon_apply_push_batched(const long long* master_ptrs, const long long* value_offsets, const PeerPtrs& values,
                                  int world, const __nv_bfloat16* xb, const float* scale0, const float* line_scale,
                                  bool lines_are_rows, int P, int rows, int cols, float lr, float weight_decay,
                                  cudaStream_t s) {
  const long long n = static_cast<long long>(rows) * cols;
  if (n <= 0 || P <= 0) return;
  int gx = grid_for(n, 8, (148 * 8 + P - 1) / P);
  muon_apply_push_batched_kernel<<<dim3(gx, P), 256, 0, s>>>(master_ptrs, value_offsets, values, world, xb, scale0,
                                                             line_scale, lines_are_rows, rows, cols, lr, weight_decay);
}

#endif  // !NC_EMU

}  // namespace nc

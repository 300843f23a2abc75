// bf16 GEMM for sm_100a: TMA -> shared memory ring -> tcgen05.mma -> TMEM -> fused epilogue.
//
//   C[b][M,N] = epilogue( sum_k A[b][m,k] * B[b][n,k] )
//
// Either operand may be stored K-major (contraction index contiguous: x and W in y = x W^T) or
// MN-major (output index contiguous: the layouts that dgrad and wgrad meet without any transpose
// copy). One persistent CTA per SM, 192 threads:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation + tcgen05.mma issue (one elected lane)
//   warps 2..5  epilogue: tcgen05.ld 32x32b -> registers -> global (each warp owns the TMEM lane
//               quadrant warp_id % 4)
// Tile 128 x 256 x 64, 4-stage ring (48 KiB per stage), two 256-column TMEM accumulators so that the
// epilogue of tile i overlaps the main loop of tile i+1. Work units are (batch, tile, k-split); k-splits
// exist only for fp32 outputs and are combined with vector red.global.add.
//
// This kernel covers what the reference spreads over cuBLAS/cublasLt calls and pointwise launches
// (reference backends/cuda/gemm.cu:474-538 and the relu^2 / residual / accumulate pointwise passes of
// src/ops.cc:551-706, 1110-1141): the epilogues below fold those passes into the GEMM.
#include "gemm_tcgen05.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "ptx.cuh"
#include "tmap.h"

namespace nc {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int CHUNK_BYTES = 64 * BK * 2;  // one 64-wide MN chunk of an MN-major tile: 8 KiB
constexpr int GROUP_M = 16;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

struct KernelParams {
  int M, N, K;
  int batch;
  int m_blocks, n_blocks, k_blocks, splits, kb_per_split;
  void* C;
  long long ldc, strideC;
  void* C2;
  const __nv_bfloat16* R;
  long long ldr, strideR;
  float alpha, beta;
  int* status;
  const int* wait_flags;
  int wait_count, wait_value;
  const uint4* gather_src;
  uint4* gather_dst;
  long long gather_vecs;
  int* gather_counter;
  int gather_base;
};

struct Unit {
  int b, m_blk, n_blk, kb0, kb1;
};

__device__ __forceinline__ Unit decode_unit(const KernelParams& p, int unit) {
  Unit u;
  // split-major: consecutive units (the ones in flight together) share a k-range, so operand panels of
  // neighbouring tiles are still shared through L2 when K is split
  const int tiles = p.batch * p.m_blocks * p.n_blocks;
  const int split = unit / tiles;
  int t = unit - split * tiles;
  const int per_batch = p.m_blocks * p.n_blocks;
  u.b = t / per_batch;
  t -= u.b * per_batch;
  const int group_size = GROUP_M * p.n_blocks;
  const int g = t / group_size;
  const int first_m = g * GROUP_M;
  const int gm = min(p.m_blocks - first_m, GROUP_M);
  const int r = t - g * group_size;
  u.m_blk = first_m + r % gm;
  u.n_blk = r / gm;
  u.kb0 = split * p.kb_per_split;
  u.kb1 = min(p.k_blocks, u.kb0 + p.kb_per_split);
  return u;
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const KernelParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_units = p.batch * p.m_blocks * p.n_blocks * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (p.gather_src != nullptr) {
    // All-gather fused into the consuming GEMM: every CTA pulls its slice of the weight from the owner's
    // memory with plain peer loads and stores it at the local address the tensor map points to.
    const long long per = (p.gather_vecs + gridDim.x - 1) / gridDim.x;
    const long long v0 = static_cast<long long>(blockIdx.x) * per;
    const long long v1 = min(p.gather_vecs, v0 + per);
    for (long long i = v0 + threadIdx.x; i < v1; i += NUM_THREADS) p.gather_dst[i] = p.gather_src[i];
    __threadfence();
    asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy stores before async-proxy (TMA) loads
    __syncthreads();
    if (threadIdx.x == 0) atomicAdd(p.gather_counter, 1);
  }

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (p.gather_src != nullptr) {
        const unsigned long long t0 = globaltimer_ns();
        const int want = p.gather_base + static_cast<int>(gridDim.x);
        while (ok && ld_acquire_sys(p.gather_counter) - want < 0) {
          if (globaltimer_ns() - t0 > kWaitBudgetNs) {
            *abort_flag = 1;
            if (p.status != nullptr) atomicCAS(p.status, 0, kErrWaitOther);
            ok = false;
          }
        }
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      if (ok && p.wait_flags != nullptr && !wait_flags_bounded(p.wait_flags, p.wait_count, p.wait_value, p.status)) {
        *abort_flag = 1;
        ok = false;
      }
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const Unit u = decode_unit(p, unit);
        for (int kb = u.kb0; kb < u.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrWaitEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_3d(sa + c * CHUNK_BYTES, &tmA, &full_bar[stage], u.m_blk * BM + c * 64, kb * BK, u.b);
          } else {
            tma_load_3d(sa, &tmA, &full_bar[stage], kb * BK, u.m_blk * BM, u.b);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_3d(sb + c * CHUNK_BYTES, &tmB, &full_bar[stage], u.n_blk * BN + c * 64, kb * BK, u.b);
          } else {
            tma_load_3d(sb, &tmB, &full_bar[stage], kb * BK, u.n_blk * BN, u.b);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Aborted: give the copies already in flight time to land before the CTA retires.
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      // per-UMMA_K advance of the start address, in 16-byte units
      constexpr int kStepA = A_MN ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
      constexpr int kStepB = B_MN ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
      const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem), A_MN ? CHUNK_BYTES : 16, 1024);
      const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(smem) + A_BYTES, B_MN ? CHUNK_BYTES : 16, 1024);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const Unit u = decode_unit(p, unit);
        if (u.kb1 <= u.kb0) continue;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, kErrWaitTmemEmpty)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = u.kb0; kb < u.kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kErrWaitFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          // descriptors differ from the stage-0 ones only in the 16-byte-unit start address field
          const uint64_t da0 = a_desc0 + static_cast<uint64_t>(stage * (STAGE_BYTES >> 4));
          const uint64_t db0 = b_desc0 + static_cast<uint64_t>(stage * (STAGE_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            mma_f16_ss(d_tmem, da0 + static_cast<uint64_t>(k * kStepA), db0 + static_cast<uint64_t>(k * kStepB), idesc,
                       (kb > u.kb0 || k > 0) ? 1u : 0u);
          }
          mma_commit(&empty_bar[stage]);  // the stage is free once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        mma_commit(&tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
      const Unit u = decode_unit(p, unit);
      if (u.kb1 <= u.kb0) continue;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, kErrWaitTmemFull)) break;
      tc_fence_after();
      const int row = u.m_blk * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const long long crow = static_cast<long long>(u.b) * p.strideC + static_cast<long long>(row) * p.ldc;
      const long long rrow = static_cast<long long>(u.b) * p.strideR + static_cast<long long>(row) * p.ldr;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        const int col0 = u.n_blk * BN + c * 32;
        if (!row_ok || col0 >= p.N) continue;
        if (EPI == kEpiF32) {
          float* crow_p = reinterpret_cast<float*>(p.C) + crow + col0;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (col0 + j * 4 >= p.N) break;
            float4 v = make_float4(__uint_as_float(r[4 * j]) * p.alpha, __uint_as_float(r[4 * j + 1]) * p.alpha,
                                   __uint_as_float(r[4 * j + 2]) * p.alpha, __uint_as_float(r[4 * j + 3]) * p.alpha);
            float4* dst = reinterpret_cast<float4*>(crow_p + j * 4);
            if (p.splits > 1) {
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z),
                           "f"(v.w)
                           : "memory");
            } else {
              if (p.beta != 0.0f) {
                const float4 o = *dst;
                v.x += p.beta * o.x;
                v.y += p.beta * o.y;
                v.z += p.beta * o.z;
                v.w += p.beta * o.w;
              }
              *dst = v;
            }
          }
        } else {
          __nv_bfloat16* crow_p = reinterpret_cast<__nv_bfloat16*>(p.C) + crow + col0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (col0 + j * 8 >= p.N) break;
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]);
            uint4 out, out2;
            if (EPI == kEpiBf16) {
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] *= p.alpha;
            } else if (EPI == kEpiBf16Res) {
              const uint4 rv = *reinterpret_cast<const uint4*>(p.R + rrow + col0 + j * 8);
              const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                f[2 * e] = p.alpha * f[2 * e] + p.beta * bf16_lo(rw[e]);
                f[2 * e + 1] = p.alpha * f[2 * e + 1] + p.beta * bf16_hi(rw[e]);
              }
            } else if (EPI == kEpiDRelu2) {
              const uint4 rv = *reinterpret_cast<const uint4*>(p.R + rrow + col0 + j * 8);
              const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                f[2 * e] *= 2.0f * fmaxf(bf16_lo(rw[e]), 0.0f);
                f[2 * e + 1] *= 2.0f * fmaxf(bf16_hi(rw[e]), 0.0f);
              }
            }
            out.x = pack_bf16(f[0], f[1]);
            out.y = pack_bf16(f[2], f[3]);
            out.z = pack_bf16(f[4], f[5]);
            out.w = pack_bf16(f[6], f[7]);
            *reinterpret_cast<uint4*>(crow_p + j * 8) = out;
            if (EPI == kEpiRelu2) {
              // act = relu(pre)^2 computed from the rounded pre-activation, as a separate pass would.
              const uint32_t ow[4] = {out.x, out.y, out.z, out.w};
              uint32_t aw[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float lo = fmaxf(bf16_lo(ow[e]), 0.0f);
                const float hi = fmaxf(bf16_hi(ow[e]), 0.0f);
                aw[e] = pack_bf16(lo * lo, hi * hi);
              }
              out2 = make_uint4(aw[0], aw[1], aw[2], aw[3]);
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C2) + crow + col0 + j * 8) = out2;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

namespace {

template <bool A_MN, bool B_MN, int EPI>
cudaError_t launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const KernelParams& kp, int grid,
                       cudaStream_t stream) {
  static bool configured = false;
  auto kernel = gemm_kernel<A_MN, B_MN, EPI>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, kp);
  return cudaGetLastError();
}

template <bool A_MN, bool B_MN>
cudaError_t launch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const KernelParams& kp, int grid,
                       cudaStream_t stream) {
  switch (epi) {
    case kEpiBf16: return launch_one<A_MN, B_MN, kEpiBf16>(ta, tb, kp, grid, stream);
    case kEpiBf16Res: return launch_one<A_MN, B_MN, kEpiBf16Res>(ta, tb, kp, grid, stream);
    case kEpiRelu2: return launch_one<A_MN, B_MN, kEpiRelu2>(ta, tb, kp, grid, stream);
    case kEpiDRelu2: return launch_one<A_MN, B_MN, kEpiDRelu2>(ta, tb, kp, grid, stream);
    case kEpiF32: return launch_one<A_MN, B_MN, kEpiF32>(ta, tb, kp, grid, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

const char* gemm_bf16(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0) return nullptr;
  if (a.lda % 8 || a.ldb % 8) return "gemm_bf16: operand leading dimensions must be multiples of 8 elements";
  if ((reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.B)) & 15)
    return "gemm_bf16: operand base addresses must be 16-byte aligned";
  if (a.batch > 1 && ((a.strideA % 8) || (a.strideB % 8))) return "gemm_bf16: batch strides must be multiples of 8";
  const bool f32 = a.epi == kEpiF32;
  if (f32 ? (a.N % 4 || a.ldc % 4) : (a.N % 8 || a.ldc % 8)) return "gemm_bf16: N and ldc must allow 16-byte stores";
  if ((a.epi == kEpiBf16Res || a.epi == kEpiDRelu2) && (a.R == nullptr || a.ldr % 8))
    return "gemm_bf16: residual operand missing or misaligned";
  if (a.epi == kEpiRelu2 && a.C2 == nullptr) return "gemm_bf16: relu2 epilogue needs the second output";

  CUtensorMap ta, tb;
  const long long sA = a.batch > 1 ? a.strideA : static_cast<long long>(a.a_mn_major ? a.K : a.M) * a.lda;
  const long long sB = a.batch > 1 ? a.strideB : static_cast<long long>(a.b_mn_major ? a.K : a.N) * a.ldb;
  bool ok = a.a_mn_major ? make_tmap_bf16_3d(&ta, a.A, a.M, a.K, a.batch, a.lda, sA, 64, BK)
                         : make_tmap_bf16_3d(&ta, a.A, a.K, a.M, a.batch, a.lda, sA, BK, BM);
  ok = ok && (a.b_mn_major ? make_tmap_bf16_3d(&tb, a.B, a.N, a.K, a.batch, a.ldb, sB, 64, BK)
                           : make_tmap_bf16_3d(&tb, a.B, a.K, a.N, a.batch, a.ldb, sB, BK, BN));
  if (!ok) return "gemm_bf16: cuTensorMapEncodeTiled failed";

  KernelParams kp;
  kp.M = a.M, kp.N = a.N, kp.K = a.K, kp.batch = a.batch;
  kp.m_blocks = (a.M + BM - 1) / BM;
  kp.n_blocks = (a.N + BN - 1) / BN;
  kp.k_blocks = (a.K + BK - 1) / BK;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  static int cached_sms[64] = {0};
  if (dev < 64 && cached_sms[dev] == 0) cudaDeviceGetAttribute(&cached_sms[dev], cudaDevAttrMultiProcessorCount, dev);
  if (dev < 64 && cached_sms[dev] > 0) sms = cached_sms[dev];
  const long long tiles = static_cast<long long>(kp.batch) * kp.m_blocks * kp.n_blocks;
  // K is split when whole tiles would leave SMs idle (fewer tiles than SMs, or a ragged last wave).
  // The split count maximises wave efficiency minus a small charge per split for the red.add traffic.
  int splits = 1;
  if (f32 && a.allow_split_k && (a.beta == 0.0f || a.beta == 1.0f)) {
    double best = -1.0;
    const int max_splits = kp.k_blocks / 16 > 0 ? (kp.k_blocks / 16 < 24 ? kp.k_blocks / 16 : 24) : 1;
    for (int s = 1; s <= max_splits; ++s) {
      const long long units = tiles * s;
      const long long waves = (units + sms - 1) / sms;
      const double score = static_cast<double>(units) / static_cast<double>(waves * sms) - 0.004 * (s - 1);
      if (score > best + 1e-9) {
        best = score;
        splits = s;
      }
    }
  }
  kp.kb_per_split = (kp.k_blocks + splits - 1) / splits;
  splits = (kp.k_blocks + kp.kb_per_split - 1) / kp.kb_per_split;  // no empty split
  kp.splits = splits;
  kp.C = a.C, kp.ldc = a.ldc, kp.strideC = a.strideC;
  kp.C2 = a.C2;
  kp.R = static_cast<const __nv_bfloat16*>(a.R), kp.ldr = a.ldr, kp.strideR = a.strideR;
  kp.alpha = a.alpha, kp.beta = a.beta;
  kp.status = a.status;
  kp.wait_flags = a.wait_flags, kp.wait_count = a.wait_count, kp.wait_value = a.wait_value;
  kp.gather_src = static_cast<const uint4*>(a.gather_src);
  kp.gather_dst = static_cast<uint4*>(const_cast<void*>(a.B));
  kp.gather_vecs = a.gather_bytes / 16;
  kp.gather_counter = a.gather_counter;
  kp.gather_base = a.gather_base;
  if (a.gather_src != nullptr && (a.gather_counter == nullptr || (a.gather_bytes % 16) != 0))
    return "gemm_bf16: gather needs a counter and a byte count that is a multiple of 16";
  if (f32 && splits > 1 && a.beta == 0.0f) {
    // red.add needs a zeroed destination
    if (a.ldc == a.N && a.batch == 1) {
      cudaMemsetAsync(a.C, 0, static_cast<size_t>(a.M) * a.N * 4, stream);
    } else {
      for (int b = 0; b < a.batch; ++b)
        cudaMemset2DAsync(static_cast<float*>(a.C) + b * a.strideC, a.ldc * 4, 0, static_cast<size_t>(a.N) * 4, a.M,
                          stream);
    }
  }
  const long long units = tiles * splits;
  const int grid = static_cast<int>(units < sms ? units : sms);
  cudaError_t e;
  if (a.a_mn_major) {
    e = a.b_mn_major ? launch_epi<true, true>(a.epi, ta, tb, kp, grid, stream)
                     : launch_epi<true, false>(a.epi, ta, tb, kp, grid, stream);
  } else {
    e = a.b_mn_major ? launch_epi<false, true>(a.epi, ta, tb, kp, grid, stream)
                     : launch_epi<false, false>(a.epi, ta, tb, kp, grid, stream);
  }
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nc

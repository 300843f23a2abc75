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
#include <cstdlib>
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
constexpr int kEpiStageBytes = 32 * 64;  // one epilogue warp's staging tile (32 rows x 32 bf16)
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/ + 4 * kEpiStageBytes;

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

// One 32-column chunk of a thread's accumulator row through the fused epilogue EPI to global memory.
// `rv` holds the thread's 32 residual / pre-activation values (bf16) for the epilogues that read R.
// One MUFU instruction; the result feeds a bf16 rounding, so the approximation error (about 1 fp32 ulp) is invisible.
__device__ __forceinline__ float sqrt_approx(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// bf16 outputs leave through a warp-private shared-memory tile: a thread owns one accumulator row (a TMEM lane), so
// storing straight from registers would scatter 16 bytes to each of 32 rows per instruction (32 half-filled
// sectors). The warp writes its 32 rows x 64 bytes to shared memory (granules swizzled against bank conflicts) and
// reads them back so that four lanes cover the 64 contiguous bytes of one row: 16 full sectors per instruction.
struct EpiWarp {
  uint8_t* stage;       // 32 rows x 64 bytes, private to the warp
  int lane;
  int rows_valid;       // rows of this warp's 32 that exist (M edge)
  long long crow0;      // element offset of the warp's first row in C (and C2)
};

__device__ __forceinline__ void emit_rows(const KernelParams& p, const EpiWarp& w, __nv_bfloat16* base, int col0,
                                          const uint4 (&out)[4], bool own_row_ok) {
  const int r = w.lane;
  if (own_row_ok) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *reinterpret_cast<uint4*>(w.stage + r * 64 + ((j ^ ((r >> 1) & 3)) << 4)) = out[j];
  }
  __syncwarp();
  const int g = w.lane & 3;
  const bool col_ok = col0 + g * 8 < p.N;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int rr = it * 8 + (w.lane >> 2);
    if (col_ok && rr < w.rows_valid) {
      const uint4 v = *reinterpret_cast<const uint4*>(w.stage + rr * 64 + ((g ^ ((rr >> 1) & 3)) << 4));
      *reinterpret_cast<uint4*>(base + w.crow0 + static_cast<long long>(rr) * p.ldc + col0 + g * 8) = v;
    }
  }
  __syncwarp();
}

template <int EPI>
__device__ __forceinline__ void store_chunk(const KernelParams& p, const uint32_t (&r)[32], const uint4 (&rv)[4],
                                            int col0, long long crow, const EpiWarp& w, bool row_ok) {
  if (EPI == kEpiF32) {
    if (!row_ok) return;
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
    return;
  }
  uint4 outs[4], acts[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]);
    const uint32_t rw[4] = {rv[j].x, rv[j].y, rv[j].z, rv[j].w};
    if (EPI == kEpiBf16) {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] *= p.alpha;
    } else if (EPI == kEpiBf16Res) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        f[2 * e] = p.alpha * f[2 * e] + p.beta * bf16_lo(rw[e]);
        f[2 * e + 1] = p.alpha * f[2 * e + 1] + p.beta * bf16_hi(rw[e]);
      }
    } else if (EPI == kEpiDRelu2) {
      // d(pre) = d(act) * 2 relu(pre). The side operand is either the saved pre-activation (beta == 0) or the saved
      // activation act = relu(pre)^2 (beta != 0), from which relu(pre) = sqrt(act).
      const bool from_act = p.beta != 0.0f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = fmaxf(bf16_lo(rw[e]), 0.0f), hi = fmaxf(bf16_hi(rw[e]), 0.0f);
        f[2 * e] *= 2.0f * (from_act ? sqrt_approx(lo) : lo);
        f[2 * e + 1] *= 2.0f * (from_act ? sqrt_approx(hi) : hi);
      }
    }
    uint4 out;
    out.x = pack_bf16(f[0], f[1]);
    out.y = pack_bf16(f[2], f[3]);
    out.z = pack_bf16(f[4], f[5]);
    out.w = pack_bf16(f[6], f[7]);
    outs[j] = out;
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
      acts[j] = make_uint4(aw[0], aw[1], aw[2], aw[3]);
    }
  }
  // relu2 with C2 == C: only the activation is kept (the backward then works from the activation alone)
  if (EPI != kEpiRelu2 || p.C != p.C2) emit_rows(p, w, reinterpret_cast<__nv_bfloat16*>(p.C), col0, outs, row_ok);
  if (EPI == kEpiRelu2) emit_rows(p, w, reinterpret_cast<__nv_bfloat16*>(p.C2), col0, acts, row_ok);
}

template <int EPI>
__device__ __forceinline__ void load_residual(const KernelParams& p, uint4 (&rv)[4], int col0, long long rrow,
                                              bool row_ok) {
  if (EPI != kEpiBf16Res && EPI != kEpiDRelu2) return;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    rv[j] = (row_ok && col0 + j * 8 < p.N) ? *reinterpret_cast<const uint4*>(p.R + rrow + col0 + j * 8)
                                           : make_uint4(0, 0, 0, 0);
  }
}

// Epilogue of one warp: its 32 accumulator rows x BN columns from TMEM (`taddr` = lane quadrant and first
// column), through the fused epilogue EPI, to global memory. `crow` / `rrow` are the element offsets of the
// thread's row in C and R. The TMEM read and the residual load of chunk c+1 are in flight while chunk c is
// converted and stored.
template <int EPI>
__device__ __forceinline__ void store_tile(const KernelParams& p, uint32_t taddr, int n_base, bool row_ok,
                                           long long crow, long long rrow, const EpiWarp& w) {
  uint32_t r0[32], r1[32];
  uint4 q0[4], q1[4];
  tmem_ld_32x32(taddr, r0);
  load_residual<EPI>(p, q0, n_base, rrow, row_ok);
#pragma unroll 1
  for (int c = 0; c < BN / 32; c += 2) {
    tmem_ld_wait();
    tmem_ld_32x32(taddr + (c + 1) * 32, r1);
    load_residual<EPI>(p, q1, n_base + (c + 1) * 32, rrow, row_ok);
    if (n_base + c * 32 < p.N) store_chunk<EPI>(p, r0, q0, n_base + c * 32, crow, w, row_ok);
    tmem_ld_wait();
    if (c + 2 < BN / 32) {
      tmem_ld_32x32(taddr + (c + 2) * 32, r0);
      load_residual<EPI>(p, q0, n_base + (c + 2) * 32, rrow, row_ok);
    }
    if (n_base + (c + 1) * 32 < p.N) store_chunk<EPI>(p, r1, q1, n_base + (c + 1) * 32, crow, w, row_ok);
  }
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
      EpiWarp w;
      w.stage = smem + STAGES * STAGE_BYTES + 256 + q * kEpiStageBytes;
      w.lane = lane;
      w.rows_valid = min(32, p.M - (row - lane));
      w.crow0 = crow - static_cast<long long>(lane) * p.ldc;
      store_tile<EPI>(p, tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16), u.n_blk * BN, row_ok, crow, rrow, w);
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

// ---------------------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs computes one 256 x 256 tile with tcgen05.mma.cta_group::2. Each CTA loads
// its 128 rows of A and its 128-column half of B (32 KiB per stage instead of 48), so the operand traffic per
// FLOP drops by a third: the single-CTA kernel is bound by shared-memory fill bandwidth, not by the tensor
// pipe. The even CTA of the pair owns the "full" barriers (both CTAs' TMA loads complete on them) and issues the
// MMAs; commits arrive on the "empty" / "accumulator full" barriers of both CTAs; both CTAs run the epilogue
// for their own 128 accumulator rows and release the accumulator to the even CTA's barrier.
constexpr int P_STAGES = 6;
constexpr int P_A_BYTES = BM * BK * 2;         // 16 KiB
constexpr int P_B_BYTES = (BN / 2) * BK * 2;   // 16 KiB: this CTA's half of the 256-wide B tile
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 + 256 + 4 * kEpiStageBytes;

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const KernelParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + P_STAGES * P_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + P_STAGES;
  uint64_t* tmem_full = empty_bar + P_STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int total_units = p.batch * p.m_blocks * p.n_blocks * p.splits;   // m_blocks counts 256-row tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);    // the leader's arrive.expect_tx; bytes of both CTAs complete on it
      mbar_init(&empty_bar[s], 1);   // one commit (delivered to both CTAs)
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);  // four epilogue warps of each CTA (used in the leader only)
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // barrier initialisation of both CTAs is visible before any remote arrive or copy
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (p.wait_flags != nullptr && !wait_flags_bounded(p.wait_flags, p.wait_count, p.wait_value, p.status)) {
        *abort_flag = 1;
        ok = false;
      }
      for (int unit = pair_id; unit < total_units && ok; unit += num_pairs) {
        const Unit u = decode_unit(p, unit);
        const int m0 = u.m_blk * (2 * BM) + static_cast<int>(rank) * BM;
        const int n0 = u.n_blk * BN + static_cast<int>(rank) * (BN / 2);
        for (int kb = u.kb0; kb < u.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrWaitEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * P_STAGE_BYTES;
          uint8_t* sb = sa + P_A_BYTES;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * P_STAGE_BYTES);
          const uint32_t bar = mapa_u32(&full_bar[stage], 0);
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_3d_pair(sa + c * CHUNK_BYTES, &tmA, bar, m0 + c * 64, kb * BK, u.b);
          } else {
            tma_load_3d_pair(sa, &tmA, bar, kb * BK, m0, u.b);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 128; ++c)
              tma_load_3d_pair(sb + c * CHUNK_BYTES, &tmB, bar, n0 + c * 64, kb * BK, u.b);
          } else {
            tma_load_3d_pair(sb, &tmB, bar, kb * BK, n0, u.b);
          }
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      constexpr int kStepA = A_MN ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
      constexpr int kStepB = B_MN ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
      const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem), A_MN ? CHUNK_BYTES : 16, 1024);
      const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(smem) + P_A_BYTES, B_MN ? CHUNK_BYTES : 16, 1024);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int unit = pair_id; unit < total_units && ok; unit += num_pairs) {
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
          const uint64_t da0 = a_desc0 + static_cast<uint64_t>(stage * (P_STAGE_BYTES >> 4));
          const uint64_t db0 = b_desc0 + static_cast<uint64_t>(stage * (P_STAGE_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            mma_f16_ss_pair(d_tmem, da0 + static_cast<uint64_t>(k * kStepA), db0 + static_cast<uint64_t>(k * kStepB),
                            idesc, (kb > u.kb0 || k > 0) ? 1u : 0u);
          }
          mma_commit_pair(&empty_bar[stage], 3);   // frees the stage in both CTAs
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        mma_commit_pair(&tmem_full[acc], 3);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t leader_empty0 = mapa_u32(&tmem_empty[0], 0);
    const uint32_t leader_empty1 = mapa_u32(&tmem_empty[1], 0);
    for (int unit = pair_id; unit < total_units; unit += num_pairs) {
      const Unit u = decode_unit(p, unit);
      if (u.kb1 <= u.kb0) continue;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, kErrWaitTmemFull)) break;
      tc_fence_after();
      const int row = u.m_blk * (2 * BM) + static_cast<int>(rank) * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const long long crow = static_cast<long long>(u.b) * p.strideC + static_cast<long long>(row) * p.ldc;
      const long long rrow = static_cast<long long>(u.b) * p.strideR + static_cast<long long>(row) * p.ldr;
      EpiWarp w;
      w.stage = smem + P_STAGES * P_STAGE_BYTES + 256 + q * kEpiStageBytes;
      w.lane = lane;
      w.rows_valid = min(32, p.M - (row - lane));
      w.crow0 = crow - static_cast<long long>(lane) * p.ldc;
      store_tile<EPI>(p, tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16), u.n_blk * BN, row_ok, crow, rrow, w);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc == 0 ? leader_empty0 : leader_empty1);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // neither CTA frees tensor memory or retires while the other may still use the pair
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
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

template <bool A_MN, bool B_MN, int EPI>
cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const KernelParams& kp, int max_pairs,
                        long long units, cudaStream_t stream) {
  static bool configured = false;
  auto kernel = gemm_pair_kernel<A_MN, B_MN, EPI>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int pairs = static_cast<int>(units < max_pairs ? units : max_pairs);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = P_SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, ta, tb, kp);
}

template <bool A_MN, bool B_MN>
cudaError_t launch_pair_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const KernelParams& kp,
                            int max_pairs, long long units, cudaStream_t stream) {
  switch (epi) {
    case kEpiBf16: return launch_pair<A_MN, B_MN, kEpiBf16>(ta, tb, kp, max_pairs, units, stream);
    case kEpiBf16Res: return launch_pair<A_MN, B_MN, kEpiBf16Res>(ta, tb, kp, max_pairs, units, stream);
    case kEpiRelu2: return launch_pair<A_MN, B_MN, kEpiRelu2>(ta, tb, kp, max_pairs, units, stream);
    case kEpiDRelu2: return launch_pair<A_MN, B_MN, kEpiDRelu2>(ta, tb, kp, max_pairs, units, stream);
    case kEpiF32: return launch_pair<A_MN, B_MN, kEpiF32>(ta, tb, kp, max_pairs, units, stream);
  }
  return cudaErrorInvalidValue;
}

// Clusters of two 1-CTA-per-SM blocks that can be resident at once on the current device.
int max_active_pairs(int dev) {
  static int cached[64] = {0};
  if (dev >= 0 && dev < 64 && cached[dev] != 0) return cached[dev] > 0 ? cached[dev] : 0;
  auto kernel = gemm_pair_kernel<false, false, kEpiBf16>;
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 148);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = P_SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = 0;
  }
  if (dev >= 0 && dev < 64) cached[dev] = n > 0 ? n : -1;
  return n;
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

  KernelParams kp;
  kp.M = a.M, kp.N = a.N, kp.K = a.K, kp.batch = a.batch;
  kp.n_blocks = (a.N + BN - 1) / BN;
  kp.k_blocks = (a.K + BK - 1) / BK;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  static int cached_sms[64] = {0};
  if (dev < 64 && cached_sms[dev] == 0) cudaDeviceGetAttribute(&cached_sms[dev], cudaDevAttrMultiProcessorCount, dev);
  if (dev < 64 && cached_sms[dev] > 0) sms = cached_sms[dev];
  // Tile shape: 256-row tiles on CTA pairs when they fill the machine about as well as 128-row tiles on single
  // CTAs (the pair kernel moves a third less operand data per FLOP).
  static const bool pair_enabled = [] {
    const char* e = std::getenv("NANOCHAT_GEMM_PAIR");
    return e == nullptr || e[0] != '0';
  }();
  const int mb1 = (a.M + BM - 1) / BM, mb2 = (a.M + 2 * BM - 1) / (2 * BM);
  const long long tiles1 = static_cast<long long>(kp.batch) * mb1 * kp.n_blocks;
  const long long tiles2 = static_cast<long long>(kp.batch) * mb2 * kp.n_blocks;
  int pairs = 0;
  bool use_pair = false;
  if (pair_enabled && a.gather_src == nullptr && a.M >= 2 * BM) {
    pairs = max_active_pairs(dev);
    if (pairs > 0) {
      auto eff = [](long long units, int slots) {
        const long long waves = (units + slots - 1) / slots;
        return static_cast<double>(units) / static_cast<double>(waves * slots);
      };
      const bool splittable = a.epi == kEpiF32 && a.allow_split_k;
      use_pair = splittable || (static_cast<double>(2 * pairs) / sms) * eff(tiles2, pairs) * 1.08 >= eff(tiles1, sms);
    }
  }
  kp.m_blocks = use_pair ? mb2 : mb1;
  const int slots = use_pair ? pairs : sms;

  CUtensorMap ta, tb;
  const long long sA = a.batch > 1 ? a.strideA : static_cast<long long>(a.a_mn_major ? a.K : a.M) * a.lda;
  const long long sB = a.batch > 1 ? a.strideB : static_cast<long long>(a.b_mn_major ? a.K : a.N) * a.ldb;
  bool ok = a.a_mn_major ? make_tmap_bf16_3d(&ta, a.A, a.M, a.K, a.batch, a.lda, sA, 64, BK)
                         : make_tmap_bf16_3d(&ta, a.A, a.K, a.M, a.batch, a.lda, sA, BK, BM);
  ok = ok && (a.b_mn_major ? make_tmap_bf16_3d(&tb, a.B, a.N, a.K, a.batch, a.ldb, sB, 64, BK)
                           : make_tmap_bf16_3d(&tb, a.B, a.K, a.N, a.batch, a.ldb, sB, BK, use_pair ? BN / 2 : BN));
  if (!ok) return "gemm_bf16: cuTensorMapEncodeTiled failed";

  const long long tiles = use_pair ? tiles2 : tiles1;
  // K is split when whole tiles would leave SMs idle (fewer tiles than SMs, or a ragged last wave).
  // The split count maximises wave efficiency minus a small charge per split for the red.add traffic.
  int splits = 1;
  if (f32 && a.allow_split_k && (a.beta == 0.0f || a.beta == 1.0f)) {
    double best = -1.0;
    const int max_splits = kp.k_blocks / 16 > 0 ? (kp.k_blocks / 16 < 24 ? kp.k_blocks / 16 : 24) : 1;
    for (int s = 1; s <= max_splits; ++s) {
      const long long units = tiles * s;
      const long long waves = (units + slots - 1) / slots;
      const double score = static_cast<double>(units) / static_cast<double>(waves * slots) - 0.004 * (s - 1);
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
  cudaError_t e;
  if (use_pair) {
    if (a.a_mn_major) {
      e = a.b_mn_major ? launch_pair_epi<true, true>(a.epi, ta, tb, kp, pairs, units, stream)
                       : launch_pair_epi<true, false>(a.epi, ta, tb, kp, pairs, units, stream);
    } else {
      e = a.b_mn_major ? launch_pair_epi<false, true>(a.epi, ta, tb, kp, pairs, units, stream)
                       : launch_pair_epi<false, false>(a.epi, ta, tb, kp, pairs, units, stream);
    }
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
  }
  const int grid = static_cast<int>(units < sms ? units : sms);
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

// Block-scaled fp8 (E4M3) GEMM for sm_100a and its quantizers.
//
// The reference scales fp8 operands per tensor and calls cublasLt (backends/cuda/kernels/fp8.cu:39-80,
// backends/cuda/gemm.cu:553-690). Here scales are fine grained - one per activation row and 128-wide K block,
// one per 128 x 128 weight block - which a single tensor-core accumulation cannot apply, so the kernel
// accumulates in two levels: tcgen05.mma (kind::f8f6f4) produces the partial product of ONE 128-deep K block in
// tensor memory, and the epilogue warps fold it into fp32 registers with the block's two scales while the tensor
// core already works on the next K block (two partial buffers of 256 columns).
//
//   warp 0       TMA producer (A 128x128 B and B 256x128 B tiles of 1-byte elements, SWIZZLE_128B)
//   warp 1       TMEM allocation + MMA issue: per K block 4 MMAs of K=32 into partial buffer p, then commit
//   warps 2..9   promotion + epilogue: warp w owns TMEM lane quadrant w%4 and the 128-column half (w-2)/4; per K
//                block: tcgen05.ld 16 columns at a time, acc += (sx * sw) * partial; at the end bf16 stores
#include "fp8.h"

#include <cuda.h>
#include <cuda_fp8.h>

#include "ptx.cuh"
#include "tmap.h"

namespace nc {

namespace {

constexpr float kE4M3Max = 448.0f;

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

// one warp per (row, 128-wide K block): 4 elements per lane
__global__ void __launch_bounds__(256) quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                            uint8_t* __restrict__ xq, float* __restrict__ scales,
                                                            int M, int K) {
  const int kbs = K / 128;
  const long long unit = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (unit >= static_cast<long long>(M) * kbs) return;
  const int row = static_cast<int>(unit / kbs), kb = static_cast<int>(unit % kbs);
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* src = x + static_cast<long long>(row) * ldx + kb * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  float v[4] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y)};
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = amax > 0.0f ? amax / kE4M3Max : 1.0f;
  const float inv = 1.0f / scale;
  uint32_t packed = 0;
#pragma unroll
  for (int e = 0; e < 4; ++e) packed |= static_cast<uint32_t>(to_e4m3(v[e] * inv)) << (8 * e);
  *reinterpret_cast<uint32_t*>(xq + static_cast<long long>(row) * K + kb * 128 + lane * 4) = packed;
  if (lane == 0) scales[static_cast<long long>(kb) * M + row] = scale;
}

// one CTA (256 threads) per 128 x 128 block
__global__ void __launch_bounds__(256) quantize_blocks_kernel(const __nv_bfloat16* __restrict__ w, long long ldw,
                                                              uint8_t* __restrict__ wq, float* __restrict__ scales,
                                                              int N, int K) {
  __shared__ float red[8];
  const int kbs = K / 128;
  const int nb = blockIdx.x / kbs, kb = blockIdx.x % kbs;
  const int t = threadIdx.x;
  // thread t handles columns (t % 32) * 4 .. +3 of rows t / 32 + 8 * i
  const int c = (t & 31) * 4, r0 = t >> 5;
  float amax = 0.0f;
  uint2 raw[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    raw[i] = *reinterpret_cast<const uint2*>(w + static_cast<long long>(nb * 128 + r0 + 8 * i) * ldw + kb * 128 + c);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(bf16_lo(raw[i].x)), fabsf(bf16_hi(raw[i].x))),
                             fmaxf(fabsf(bf16_lo(raw[i].y)), fabsf(bf16_hi(raw[i].y)))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((t & 31) == 0) red[t >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float scale = amax > 0.0f ? amax / kE4M3Max : 1.0f;
  const float inv = 1.0f / scale;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float v[4] = {bf16_lo(raw[i].x), bf16_hi(raw[i].x), bf16_lo(raw[i].y), bf16_hi(raw[i].y)};
    uint32_t packed = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) packed |= static_cast<uint32_t>(to_e4m3(v[e] * inv)) << (8 * e);
    *reinterpret_cast<uint32_t*>(wq + static_cast<long long>(nb * 128 + r0 + 8 * i) * K + kb * 128 + c) = packed;
  }
  if (t == 0) scales[static_cast<long long>(nb) * kbs + kb] = scale;
}

// ---------------------------------------------------------------------------------------------------------
constexpr int BM = 128, BN = 256, BK = 128;   // BK in elements = bytes
constexpr int UMMA_K = 32;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_WARPS = 8;
constexpr int NUM_THREADS = 64 + EPI_WARPS * 32;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct Params {
  int M, N, K, m_blocks, n_blocks, k_blocks;
  const float* scale_a;
  const float* scale_b;
  __nv_bfloat16* C;
  __nv_bfloat16* C2;
  long long ldc;
  int* status;
};

__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

template <bool RELU2>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* part_full = empty_bar + STAGES;
  uint64_t* part_empty = part_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(part_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_units = p.m_blocks * p.n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&part_full[a], 1);
      mbar_init(&part_empty[a], EPI_WARPS);
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

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const int m_blk = unit % p.m_blocks, n_blk = unit / p.m_blocks;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrWaitEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * BK, m_blk * BM);
          tma_load_2d(sa + A_BYTES, &tmB, &full_bar[stage], kb * BK, n_blk * BN);
          if (++stage == STAGES) {
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
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_e4m3(BM, BN);
      const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem), 16, 1024);
      const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(smem) + A_BYTES, 16, 1024);
      int stage = 0, pb = 0;
      uint32_t phase = 0, pphase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&part_empty[pb], pphase ^ 1, abort_flag, p.status, kErrWaitTmemEmpty) ||
              !mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kErrWaitFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t da = a_desc0 + static_cast<uint64_t>(stage * (STAGE_BYTES >> 4));
          const uint64_t db = b_desc0 + static_cast<uint64_t>(stage * (STAGE_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)   // 32 one-byte elements = 32 bytes = 2 descriptor units per step
            mma_f8_ss(tmem_base + pb * BN, da + static_cast<uint64_t>(2 * k), db + static_cast<uint64_t>(2 * k), idesc,
                      k > 0 ? 1u : 0u);
          mma_commit(&empty_bar[stage]);
          mma_commit(&part_full[pb]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
          if (++pb == 2) {
            pb = 0;
            pphase ^= 1;
          }
        }
      }
    }
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    const int kbs = p.k_blocks;
    int pb = 0;
    uint32_t pphase = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
      const int m_blk = unit % p.m_blocks, n_blk = unit / p.m_blocks;
      const int row = m_blk * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const int nb = n_blk * 2 + half;                       // 128-column scale block of this warp's half
      const bool nb_ok = nb * 128 < p.N;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
      float sa_next = row_ok ? p.scale_a[row] : 0.0f;
      float sb_next = nb_ok ? p.scale_b[static_cast<long long>(nb) * kbs] : 0.0f;
      for (int kb = 0; kb < kbs; ++kb) {
        const float sc = sa_next * sb_next;
        if (kb + 1 < kbs) {
          sa_next = row_ok ? p.scale_a[static_cast<long long>(kb + 1) * p.M + row] : 0.0f;
          sb_next = nb_ok ? p.scale_b[static_cast<long long>(nb) * kbs + kb + 1] : 0.0f;
        }
        if (!mbar_wait(&part_full[pb], pphase, abort_flag, p.status, kErrWaitTmemFull)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + pb * BN + half * 128 + (static_cast<uint32_t>(q * 32) << 16);
        uint32_t r0[16], r1[16];
        tmem_ld_32x16(taddr, r0);
#pragma unroll
        for (int c = 0; c < 8; c += 2) {
          tmem_ld_wait();
          tmem_ld_32x16(taddr + (c + 1) * 16, r1);
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c * 16 + j] = fmaf(sc, __uint_as_float(r0[j]), acc[c * 16 + j]);
          tmem_ld_wait();
          if (c + 2 < 8) tmem_ld_32x16(taddr + (c + 2) * 16, r0);
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[(c + 1) * 16 + j] = fmaf(sc, __uint_as_float(r1[j]), acc[(c + 1) * 16 + j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&part_empty[pb]);
        if (++pb == 2) {
          pb = 0;
          pphase ^= 1;
        }
      }
      if (!ok) break;
      if (row_ok) {
        const int col0 = n_blk * BN + half * 128;
        __nv_bfloat16* crow = p.C + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (col0 + j * 8 >= p.N) break;
          uint4 out;
          out.x = pack_bf16(acc[8 * j], acc[8 * j + 1]);
          out.y = pack_bf16(acc[8 * j + 2], acc[8 * j + 3]);
          out.z = pack_bf16(acc[8 * j + 4], acc[8 * j + 5]);
          out.w = pack_bf16(acc[8 * j + 6], acc[8 * j + 7]);
          *reinterpret_cast<uint4*>(crow + j * 8) = out;
          if (RELU2) {
            const uint32_t ow[4] = {out.x, out.y, out.z, out.w};
            uint32_t aw[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float lo = fmaxf(bf16_lo(ow[e]), 0.0f), hi = fmaxf(bf16_hi(ow[e]), 0.0f);
              aw[e] = pack_bf16(lo * lo, hi * hi);
            }
            *reinterpret_cast<uint4*>(p.C2 + static_cast<long long>(row) * p.ldc + col0 + j * 8) =
                make_uint4(aw[0], aw[1], aw[2], aw[3]);
          }
        }
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

void quantize_rows_1x128(const __nv_bfloat16* x, long long ldx, uint8_t* xq, float* scales, int M, int K,
                         cudaStream_t s) {
  const long long units = static_cast<long long>(M) * (K / 128);
  if (units <= 0) return;
  quantize_rows_kernel<<<static_cast<unsigned>((units + 7) / 8), 256, 0, s>>>(x, ldx, xq, scales, M, K);
}
void quantize_blocks_128x128(const __nv_bfloat16* w, long long ldw, uint8_t* wq, float* scales, int N, int K,
                             cudaStream_t s) {
  const int blocks = (N / 128) * (K / 128);
  if (blocks <= 0) return;
  quantize_blocks_kernel<<<blocks, 256, 0, s>>>(w, ldw, wq, scales, N, K);
}

const char* gemm_fp8_blockscaled(const Fp8GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return nullptr;
  if (a.K % 128) return "gemm_fp8: K must be a multiple of 128";
  if (a.N % 8 || a.ldc % 8) return "gemm_fp8: N and ldc must allow 16-byte stores";
  if ((reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.B)) & 15) return "gemm_fp8: misaligned operand";
  CUtensorMap ta, tb;
  if (!make_tmap_u8_2d(&ta, a.A, a.K, a.M, a.K, BK, BM) || !make_tmap_u8_2d(&tb, a.B, a.K, a.N, a.K, BK, BN))
    return "gemm_fp8: cuTensorMapEncodeTiled failed";
  Params p;
  p.M = a.M, p.N = a.N, p.K = a.K;
  p.m_blocks = (a.M + BM - 1) / BM, p.n_blocks = (a.N + BN - 1) / BN, p.k_blocks = a.K / BK;
  p.scale_a = a.scale_a, p.scale_b = a.scale_b;
  p.C = a.C, p.C2 = a.C2, p.ldc = a.ldc, p.status = a.status;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int units = p.m_blocks * p.n_blocks;
  const int grid = units < sms ? units : sms;
  cudaError_t e;
  if (a.C2 != nullptr) {
    static bool cfg2 = false;
    if (!cfg2) {
      cudaFuncSetAttribute(gemm_fp8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      cfg2 = true;
    }
    gemm_fp8_kernel<true><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  } else {
    static bool cfg1 = false;
    if (!cfg1) {
      cudaFuncSetAttribute(gemm_fp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      cfg1 = true;
    }
    gemm_fp8_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nc

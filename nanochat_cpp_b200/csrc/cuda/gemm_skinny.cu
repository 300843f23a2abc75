// Skinny bf16 GEMM for decode: few rows of activations (M <= 64) against a large weight matrix.
//
//   out[M, N] = epilogue( x[M, K] . w[N, K]^T )
//
// With M this small the job is to stream the weights once at full memory bandwidth, which needs every SM busy
// even when N / 128 is a handful of tiles. So the roles are swapped - the weight rows fill the 128 lanes of the
// MMA (UMMA M = 128), the tokens are its N = 64 - and K is split across the CTAs of a thread-block cluster:
// each CTA streams its K slice of the 128 weight rows through a TMA ring into tcgen05.mma, parks its fp32 partial
// tile in its own shared memory, and after a cluster barrier the first CTA of the cluster sums the partials
// through distributed shared memory, applies the epilogue and stores the (transposed) tile.
// The reference runs decode through per-row cuBLAS calls (src/generate.cc:266-412); there is no counterpart kernel.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "gemm_tcgen05.h"
#include "pdl_launch.h"
#include "ptx.cuh"
#include "tmap.h"

namespace nc {

namespace {

constexpr int TW = 128;   // weight rows per tile (MMA M)
constexpr int TX = 64;    // token rows per tile (MMA N)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int W_BYTES = TW * BK * 2, X_BYTES = TX * BK * 2, STAGE_BYTES = W_BYTES + X_BYTES;
constexpr int PART_BYTES = TX * TW * 4;   // fp32 partial tile [token][weight row]
constexpr int SMEM_BYTES = (STAGES * STAGE_BYTES > PART_BYTES ? STAGES * STAGE_BYTES : PART_BYTES) + 1024 + 256;
constexpr int NUM_THREADS = 192;

struct SkinnyParams {
  int M, N, K, k_blocks, kb_per_cta, splits;
  __nv_bfloat16* C;
  __nv_bfloat16* C2;
  const __nv_bfloat16* R;
  long long ldc, ldr;
  int epi;
  int* status;
  int early_w;   // weight tiles may be requested before the previous kernel of the stream has finished
};

__device__ __forceinline__ float ld_dsmem_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const SkinnyParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + SMEM_BYTES - 1024 - 256);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* part = reinterpret_cast<float*>(smem);   // reuses the ring once the MMAs have drained it

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = p.splits > 1 ? static_cast<int>(cluster_ctarank()) : 0;
  const int tile = blockIdx.x / p.splits;
  const int n0 = tile * TW;
  const int kb0 = split * p.kb_per_cta;
  const int kb1 = min(p.k_blocks, kb0 + p.kb_per_cta);
  const int my_kbs = max(kb1 - kb0, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above overlapped the tail of the previous kernel; its outputs (x, the residual) are read below, after
  // pdl_wait. With `early_w` (decode: the weights are not written by anything in the step) the producer also requests
  // the weight tiles of its first ring-full of K blocks before waiting, so most of the weight stream of a short K
  // overlaps the previous kernel as well; the x tiles of those stages follow after the wait, on the same barriers.
  int early = 0;
  if (warp == 0 && lane == 0 && p.early_w) {
    early = min(STAGES, my_kbs);
    for (int i = 0; i < early; ++i) {
      mbar_expect_tx(&full_bar[i], STAGE_BYTES);
      tma_load_3d(smem + i * STAGE_BYTES, &tmW, &full_bar[i], (kb0 + i) * BK, n0, 0);
    }
  }
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < early; ++i)
        tma_load_3d(smem + i * STAGE_BYTES + W_BYTES, &tmX, &full_bar[i], (kb0 + i) * BK, 0, 0);
      int stage = early == STAGES ? 0 : early;
      uint32_t phase = early == STAGES ? 1 : 0;
      for (int kb = kb0 + early; kb < kb1; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrWaitEmpty)) break;
        uint8_t* sw = smem + stage * STAGE_BYTES;
        mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
        tma_load_3d(sw, &tmW, &full_bar[stage], kb * BK, n0, 0);
        tma_load_3d(sw + W_BYTES, &tmX, &full_bar[stage], kb * BK, 0, 0);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && my_kbs > 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TW, TX, false, false);
      const uint64_t w_desc0 = make_smem_desc_sw128(smem_u32(smem), 16, 1024);
      const uint64_t x_desc0 = make_smem_desc_sw128(smem_u32(smem) + W_BYTES, 16, 1024);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kErrWaitFull)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t dw = w_desc0 + static_cast<uint64_t>(stage * (STAGE_BYTES >> 4));
        const uint64_t dx = x_desc0 + static_cast<uint64_t>(stage * (STAGE_BYTES >> 4));
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          mma_f16_ss(tmem_base, dw + static_cast<uint64_t>(2 * k), dx + static_cast<uint64_t>(2 * k), idesc,
                     (kb > kb0 || k > 0) ? 1u : 0u);
        mma_commit(&empty_bar[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) mma_commit(acc_full);
    }
  }

  // ---- every thread: wait for the accumulator (epilogue warps read it), exchange partials, store
  float acc[TX];
#pragma unroll
  for (int i = 0; i < TX; ++i) acc[i] = 0.0f;
  const int q = warp & 3;
  const int wrow = q * 32 + lane;   // weight row inside the tile (epilogue warps 2..5 cover quadrants 2,3,0,1)
  if (warp >= 2 && my_kbs > 0) {
    if (mbar_wait(acc_full, 0, abort_flag, p.status, kErrWaitTmemFull)) {
      tc_fence_after();
      uint32_t r[32];
#pragma unroll
      for (int c = 0; c < TX / 32; ++c) {
        tmem_ld_32x32(tmem_base + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c * 32 + j] = __uint_as_float(r[j]);
      }
    }
  }
  if (p.splits > 1) {
    __syncthreads();   // the ring is drained (acc_full implies every MMA has read its stage) before it is reused
    if (warp >= 2 && split != 0) {
#pragma unroll
      for (int m = 0; m < TX; ++m) part[m * TW + wrow] = acc[m];
    }
    cluster_sync_all();   // partials of all CTAs are in their shared memory
    if (warp >= 2 && split == 0) {
      for (int r = 1; r < p.splits; ++r) {
        const uint32_t base = mapa_u32(part, static_cast<uint32_t>(r));
#pragma unroll
        for (int m = 0; m < TX; ++m) acc[m] += ld_dsmem_f32(base + static_cast<uint32_t>((m * TW + wrow) * 4));
      }
    }
  }
  if (warp >= 2 && split == 0) {
    const int n = n0 + wrow;
    if (n < p.N) {
      // The residual may be the output itself (x += ...), so the compiler cannot move a residual load above the
      // store of the row before it: loaded inside the store loop, the 64 loads run one memory latency after the
      // other (tens of microseconds). All of them are issued here, before the first store.
      if (p.epi == kEpiBf16Res) {
        __nv_bfloat16 res[TX];
#pragma unroll
        for (int m = 0; m < TX; ++m)
          res[m] = m < p.M ? p.R[static_cast<long long>(m) * p.ldr + n] : __float2bfloat16_rn(0.0f);
#pragma unroll
        for (int m = 0; m < TX; ++m) acc[m] += __bfloat162float(res[m]);
      }
#pragma unroll
      for (int m = 0; m < TX; ++m) {   // fully unrolled: acc[] stays in registers
        if (m >= p.M) break;
        const float v = acc[m];
        const long long ci = static_cast<long long>(m) * p.ldc + n;
        const __nv_bfloat16 o = __float2bfloat16_rn(v);
        if (p.epi != kEpiRelu2 || p.C != p.C2) p.C[ci] = o;  // C2 == C: only the activation is kept
        if (p.epi == kEpiRelu2) {
          const float a = fmaxf(__bfloat162float(o), 0.0f);
          p.C2[ci] = __float2bfloat16_rn(a * a);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (p.splits > 1) cluster_sync_all();   // peers keep their shared memory alive until the sum has been read
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 64);
  }
}

}  // namespace

// Same contract as gemm_bf16 for the cases it accepts: K-major operands, batch 1, M <= 64, epilogues bf16 /
// bf16+residual (alpha = beta = 1) / relu^2. Returns nullptr on success, a message otherwise.
const char* gemm_skinny(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return nullptr;
  if (a.M > TX || a.a_mn_major || a.b_mn_major || a.batch != 1) return "gemm_skinny: unsupported operand form";
  if (a.epi != kEpiBf16 && a.epi != kEpiBf16Res && a.epi != kEpiRelu2) return "gemm_skinny: unsupported epilogue";
  if (a.lda % 8 || a.ldb % 8 || ((reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.B)) & 15))
    return "gemm_skinny: operands must be 16-byte aligned with leading dimensions in multiples of 8";
  CUtensorMap tw, tx;
  if (!make_tmap_bf16_3d(&tw, a.B, a.K, a.N, 1, a.ldb, static_cast<long long>(a.N) * a.ldb, BK, TW) ||
      !make_tmap_bf16_3d(&tx, a.A, a.K, a.M, 1, a.lda, static_cast<long long>(a.M) * a.lda, BK, TX))
    return "gemm_skinny: cuTensorMapEncodeTiled failed";
  SkinnyParams p;
  p.M = a.M, p.N = a.N, p.K = a.K;
  p.k_blocks = (a.K + BK - 1) / BK;
  const int tiles = (a.N + TW - 1) / TW;
  int splits = 1;
  // Measured on B200 (M = 64): the leader's sum over distributed shared memory costs more than it saves unless every
  // CTA of the cluster still streams about ten K blocks: 2 CTAs for K = 1280, 8 for K = 5120.
  while (splits < 8 && tiles * splits * 2 <= 592 && p.k_blocks / (splits * 2) >= 10) splits *= 2;
  if (const char* e = std::getenv("NANOCHAT_SKINNY_SPLITS")) {   // experiments: force the cluster size (1, 2, 4, 8)
    const int f = std::atoi(e);
    if (f == 1 || f == 2 || f == 4 || f == 8) splits = f;
  }
  p.splits = splits;
  p.kb_per_cta = (p.k_blocks + splits - 1) / splits;
  p.C = static_cast<__nv_bfloat16*>(a.C), p.C2 = static_cast<__nv_bfloat16*>(a.C2);
  p.R = static_cast<const __nv_bfloat16*>(a.R);
  p.ldc = a.ldc, p.ldr = a.ldr, p.epi = a.epi, p.status = a.status;
  p.early_w = pdl_enabled() ? 1 : 0;   // the inference engine turns this on around a decode step (static weights)
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * splits);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // the kernel's preamble may overlap the previous kernel of the stream (it waits before its first dependent read)
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  static const bool pdl = std::getenv("NANOCHAT_NO_PDL") == nullptr;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_skinny_kernel, tw, tx, p);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nc

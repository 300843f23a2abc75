// dQ = dS K as a banded GEMM over the dS^T tiles that the dK/dV kernel stored.
//
// The two-kernel backward used to recompute scores, probabilities and dS a second time for dQ (two extra tensor-core
// products and the whole softmax arithmetic). With dS^T [B, H, Tk, Tq] in a scratch buffer the dQ pass is pure
// streaming: one CTA per (128 query rows, head, batch) walks the 64-key sub-tiles of its band,
//     dQ[128 q, D] += dS[128 q, 64 keys] . K[64 keys, D]
// A = the stored dS^T tile read MN-major (queries contiguous), B = the K tile read MN-major (head dim contiguous):
// no transposes anywhere. A (query sub-tile, key tile) block that the dK/dV kernel did not visit holds no allowed
// pair, so its dS is exactly zero: the TMA load is pointed outside the tensor and delivers zeros.
#include <cuda.h>
#include <cuda_bf16.h>

#include "attention.h"
#include "ptx.cuh"
#include "tmap.h"

namespace nc {

namespace {

constexpr int BQ = 128;   // query rows per CTA
constexpr int BKEY = 64;  // keys per step
constexpr int STAGES = 3;
constexpr int NUM_THREADS = 192;

template <int D>
struct DqSmem {
  static constexpr int kA = BKEY * BQ * 2;   // dS^T sub-tile: two [64 keys x 64 q] chunks
  static constexpr int kB = BKEY * D * 2;    // K sub-tile: D/64 chunks of [64 keys x 64 d]
  static constexpr int kStage = kA + kB;
  static constexpr int kTotal = STAGES * kStage + 1024 + 256;
};

struct DqParams {
  int B, H, KVH, Tq, Tk, q_offset, window_left;
  int ds_tk;
  __nv_bfloat16* dq;
  long long stride_b, stride_t, stride_h;
  int* status;
};

template <int D>
__global__ void __launch_bounds__(NUM_THREADS, 2)
attention_dq_kernel(const __grid_constant__ CUtensorMap tmDS, const __grid_constant__ CUtensorMap tmK,
                    const DqParams p) {
  using L = DqSmem<D>;
  constexpr int DC = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * L::kStage);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = (p.Tq + BQ - 1) / BQ;
  const int q0 = (q_tiles - 1 - static_cast<int>(blockIdx.x)) * BQ;   // long bands first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.H / p.KVH);
  // key sub-tiles of this query tile's band
  const int q_first = p.q_offset + q0;
  const int q_last = p.q_offset + min(q0 + BQ - 1, p.Tq - 1);
  const int lo = p.window_left >= 0 ? max(0, q_first - p.window_left) : 0;
  const int j_lo = lo / BKEY;
  const int j_hi = min(q_last, p.Tk - 1) / BKEY;
  const int n_iters = max(0, j_hi - j_lo + 1);

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
    tma_prefetch_desc(&tmDS);
    tma_prefetch_desc(&tmK);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, D);
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
      for (int it = 0; it < n_iters; ++it) {
        const int j = j_lo + it;
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrWaitEmpty)) break;
        uint8_t* sa = smem + stage * L::kStage;
        uint8_t* sb = sa + L::kA;
        mbar_expect_tx(&full_bar[stage], L::kStage);
        // which 64-row query sub-tiles did the dK/dV CTA of key tile j/2 visit?
        const int kt0 = (j / 2) * 128;
        const int k_last = min(kt0 + 127, p.Tk - 1);
        const int vlo = max(0, kt0 - p.q_offset);
        int vhi = p.Tq - 1;
        if (p.window_left >= 0) vhi = min(vhi, k_last + p.window_left - p.q_offset);
        const int s_lo = vlo / 64, s_hi = vhi >= vlo ? vhi / 64 : s_lo - 1;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int s = q0 / 64 + c;
          const bool visited = s >= s_lo && s <= s_hi;
          // an unvisited block is all zeros: load from beyond the last key row (zero fill)
          tma_load_4d(sa + c * (BKEY * 128), &tmDS, &full_bar[stage], q0 + c * 64, visited ? j * BKEY : p.ds_tk, h, b);
        }
#pragma unroll
        for (int c = 0; c < DC; ++c)
          tma_load_4d(sb + c * (BKEY * 128), &tmK, &full_bar[stage], c * 64, kvh, j * BKEY, b);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_iters > 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BQ, D, true, true);   // both operands MN-major
      const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem), BKEY * 128, 1024);
      const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(smem) + L::kA, BKEY * 128, 1024);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int it = 0; it < n_iters && ok; ++it) {
        if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kErrWaitFull)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t da = a_desc0 + static_cast<uint64_t>(stage * (L::kStage >> 4));
        const uint64_t db = b_desc0 + static_cast<uint64_t>(stage * (L::kStage >> 4));
#pragma unroll
        for (int k = 0; k < BKEY / 16; ++k)   // 16 key rows of 128 bytes per step
          mma_f16_ss(tmem_base, da + static_cast<uint64_t>((k * 16 * 128) >> 4),
                     db + static_cast<uint64_t>((k * 16 * 128) >> 4), idesc, (it > 0 || k > 0) ? 1u : 0u);
        mma_commit(&empty_bar[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) mma_commit(acc_full);
    }
  } else {
    const int q = warp & 3;
    const int row = q0 + q * 32 + lane;
    bool ok = true;
    if (n_iters > 0) ok = mbar_wait(acc_full, 0, abort_flag, p.status, kErrWaitTmemFull);
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* op = p.dq + b * p.stride_b + static_cast<long long>(row) * p.stride_t + h * p.stride_h;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        if (n_iters > 0) {
          tmem_ld_32x32(tmem_base + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0u;
        }
        if (row < p.Tq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              w[e] = pack_bf16(__uint_as_float(r[g * 8 + e * 2]), __uint_as_float(r[g * 8 + e * 2 + 1]));
            *reinterpret_cast<uint4*>(op + c * 32 + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, D);
  }
}

template <int D>
const char* launch_dq(const CUtensorMap& tds, const CUtensorMap& tk, const DqParams& p, dim3 grid, cudaStream_t s) {
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(attention_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         DqSmem<D>::kTotal);
    if (e != cudaSuccess) return cudaGetErrorString(e);
    cfg = true;
  }
  attention_dq_kernel<D><<<grid, NUM_THREADS, DqSmem<D>::kTotal, s>>>(tds, tk, p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace

const char* attention_dq_from_ds(const AttnArgs& a, cudaStream_t stream) {
  CUtensorMap tds, tk;
  // dS^T [B, H, ds_tk, ds_tq]: boxes of 64 queries x 64 keys
  const long long dds[4] = {a.ds_tq, a.ds_tk, a.H, a.B};
  const long long sds[3] = {a.ds_tq, a.ds_tq * a.ds_tk, a.ds_tq * a.ds_tk * a.H};
  const int box_ds[4] = {64, BKEY, 1, 1};
  const long long dk[4] = {a.D, a.KVH, a.Tk, a.B};
  const long long sk[3] = {a.k_stride_h, a.k_stride_t, a.k_stride_b};
  const int box_k[4] = {64, 1, BKEY, 1};
  if (!make_tmap_bf16_4d(&tds, a.dS, dds, sds, box_ds) || !make_tmap_bf16_4d(&tk, a.K, dk, sk, box_k))
    return "attention_dq: tensor map construction failed";
  DqParams p;
  p.B = a.B, p.H = a.H, p.KVH = a.KVH, p.Tq = a.Tq, p.Tk = a.Tk;
  p.q_offset = a.q_offset, p.window_left = a.window_left;
  p.ds_tk = static_cast<int>(a.ds_tk);
  p.dq = static_cast<__nv_bfloat16*>(a.dQ);
  p.stride_b = a.dq_stride_b, p.stride_t = a.dq_stride_t, p.stride_h = a.dq_stride_h;
  p.status = a.status;
  const dim3 grid((a.Tq + BQ - 1) / BQ, a.H, a.B);
  return a.D == 128 ? launch_dq<128>(tds, tk, p, grid, stream) : launch_dq<64>(tds, tk, p, grid, stream);
}

}  // namespace nc

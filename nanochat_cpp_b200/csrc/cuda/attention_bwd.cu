// Sliding-window GQA flash attention, backward, for sm_100a: three launches, no atomics.
//
//   1. delta[b,h,t] = sum_d dO * O                           (row kernel)
//   2. dK, dV: one CTA per (128-key tile, kv head, batch) sweeps the 64-row query sub-tiles of every
//      query head of the group that can see the tile (the GQA fold of the reference's KeyValueGrad
//      kernel, backends/cuda/kernels/attention_flash.cu:979, without its mma.sync tiles)
//   3. dQ: one CTA per (128-row query tile, head, batch) sweeps the 64-key sub-tiles of its band
//
// Launches 2 and 3 are one kernel template. Both keep a "primary" 128-row operand pair resident in
// shared memory (K,V or Q,dO), stream 64-row "secondary" tiles (Q,dO or K,V) through a 3-stage TMA
// ring, and run per secondary tile
//      T1 = X1 * Y1^T   (scores, or scores transposed)        tcgen05.mma -> TMEM, double buffered
//      T2 = X2 * Y2^T   (dP, or dP transposed)                tcgen05.mma -> TMEM, double buffered
//      p  = exp2(T1 * c - lse),  ds = p * (T2 - delta) * scale  by 8 (dQ) or 16 (dK,dV) warps       
//      acc1 += ds * Y1  (dQ += dS K   |  dK += dS^T Q)        A = ds from shared memory,
//      acc2 += p  * Y2  (             |  dV += P^T dO)        B = the SAME shared-memory tile re-read
//                                                             through an MN-major descriptor
// so nothing is transposed in memory and the probabilities are recomputed, never stored.
#include <cuda.h>

#include <algorithm>
#include <cuda_bf16.h>

#include "attention.h"
#include "ptx.cuh"
#include "tmap.h"

namespace nc {

namespace {

constexpr int BP = 128;  // primary rows per CTA (TMEM lanes)
constexpr int BS = 64;   // secondary rows per step
// Compute warps: a multiple of four (one per TMEM lane quadrant); the warps of a quadrant split the 64 columns of
// a score tile. The dK/dV sweep is bound by the latency of its per-element chain (TMEM load, exp2, pack, stores),
// not by issue slots, so it runs four warps per scheduler; the dQ sweep keeps two.
template <int MODE>
struct BwdWarps {
  static constexpr int kCompute = MODE == 1 ? 16 : 8;
  static constexpr int kThreads = 64 + kCompute * 32;
  static constexpr int kCols = 64 / (kCompute / 4);  // score-tile columns per warp
};
constexpr int YSTAGES = 3;

enum { kModeDQ = 0, kModeDKV = 1 };

template <int D, int MODE>
struct BwdSmem {
  static constexpr int kX = BP * D * 2;       // one primary operand
  static constexpr int kY = BS * D * 2;       // one secondary operand
  static constexpr int kW = BP * BS * 2;      // one ds (or p) tile
  static constexpr int kNW = MODE == kModeDKV ? 2 : 1;
  static constexpr int kOffX1 = 0;
  static constexpr int kOffX2 = kX;
  static constexpr int kOffY = 2 * kX;                       // YSTAGES x (Y1, Y2)
  static constexpr int kOffW = kOffY + YSTAGES * 2 * kY;     // 2 buffers x kNW tiles
  static constexpr int kOffStats = kOffW + 2 * kNW * kW;     // 2 buffers x (lse2[64], delta[64])
  static constexpr int kOffBar = kOffStats + 2 * 2 * BS * 4;
  static constexpr int kTotal = kOffBar + 256 + 1024;
};

struct BwdParams {
  int B, H, KVH, Tq, Tk;
  int q_offset, window_left;
  float scale, scale_log2;
  const float* lse;    // [B, H, Tq] natural log
  const float* delta;  // [B, H, Tq]
  __nv_bfloat16* out1;  // dQ | dK
  __nv_bfloat16* out2;  //    | dV
  long long o1_stride_b, o1_stride_t, o1_stride_h;
  long long o2_stride_b, o2_stride_t, o2_stride_h;
  __nv_bfloat16* ds_out;       // DKV mode, optional: dS^T [B, H, ds_tk, ds_tq]
  long long ds_tk, ds_tq;
  int* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// tmX1/tmY1 and tmX2/tmY2: DQ mode -> X = (Q, dO), Y = (K, V); DKV mode -> X = (K, V), Y = (Q, dO).
template <int D, int MODE>
__global__ void __launch_bounds__(BwdWarps<MODE>::kThreads, 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmX2,
                     const __grid_constant__ CUtensorMap tmY1, const __grid_constant__ CUtensorMap tmY2,
                     const __grid_constant__ CUtensorMap tmDS, const BwdParams p) {
  using L = BwdSmem<D, MODE>;
  constexpr int DC = D / 64;
  constexpr int NW = L::kNW;
  constexpr int NUM_COMPUTE_WARPS = BwdWarps<MODE>::kCompute;
  constexpr int CW = BwdWarps<MODE>::kCols;
  // dK/dV sweep: the probabilities never touch shared memory. Each warp packs its 16 columns of P to bf16 and
  // stores them back over the first 8 of its own 16 score columns in TMEM; the dV product then takes its A operand
  // from TMEM (one K=16 slice per warp column group). The score buffer is rewritten by the score MMA two tiles
  // later, which the MMA thread issues after the accumulate MMAs that read P, and MMAs run in issue order.
  constexpr bool P_IN_TMEM = MODE == kModeDKV && CW == 16;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* x_full = bars + 0;
  uint64_t* y_full = bars + 1;    // [3]
  uint64_t* y_empty = bars + 4;   // [3]
  uint64_t* t_full = bars + 7;    // [2]
  uint64_t* t_empty = bars + 9;   // [2]
  uint64_t* w_full = bars + 11;   // [2]
  uint64_t* w_empty = bars + 13;  // [2]
  uint64_t* acc_full = bars + 15;
  uint64_t* stats_full = bars + 16;  // [2], one arrival per compute thread
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stats = reinterpret_cast<float*>(smem + L::kOffStats);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = p.H / p.KVH;
  const int b = blockIdx.z;
  const int p_tiles = ((MODE == kModeDQ ? p.Tq : p.Tk) + BP - 1) / BP;
  const int p_tile = MODE == kModeDQ ? (p_tiles - 1 - blockIdx.x) : blockIdx.x;
  const int p0 = p_tile * BP;  // first primary row (query row for DQ, key for DKV)
  const int hp = blockIdx.y;   // query head (DQ) or kv head (DKV)
  const int kvh = MODE == kModeDQ ? hp / group : hp;

  // secondary sub-tile range [s_lo, s_hi] (indices of 64-row tiles) and iteration count
  int s_lo, s_hi;
  if (MODE == kModeDQ) {
    const int q_first = p.q_offset + p0;
    const int q_last = p.q_offset + min(p0 + BP - 1, p.Tq - 1);
    const int lo = p.window_left >= 0 ? max(0, q_first - p.window_left) : 0;
    s_lo = lo / BS;
    s_hi = min(q_last, p.Tk - 1) / BS;
  } else {
    const int k_first = p0;
    const int k_last = min(p0 + BP - 1, p.Tk - 1);
    const int lo = max(0, k_first - p.q_offset);  // first query row whose position >= k_first
    int hi = p.Tq - 1;
    if (p.window_left >= 0) hi = min(hi, k_last + p.window_left - p.q_offset);
    s_lo = lo / BS;
    s_hi = hi >= lo ? hi / BS : s_lo - 1;
  }
  const int n_sub = max(0, s_hi - s_lo + 1);
  const int n_iters = MODE == kModeDQ ? n_sub : n_sub * group;
  // dK/dV sweep with a dS^T scratch: each finished dS tile leaves shared memory as one TMA store (its swizzled
  // K-major layout is the store's box layout), and a tile buffer is free again when the MMAs that read it have
  // completed AND the store has read it: two arrivals on w_empty.
  const bool store_ds = MODE == kModeDKV && p.ds_out != nullptr;

  if (threadIdx.x == 0) {
    mbar_init(x_full, 1);
    for (int i = 0; i < YSTAGES; ++i) {
      mbar_init(&y_full[i], 1);
      mbar_init(&y_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&t_full[i], 1);
      mbar_init(&t_empty[i], NUM_COMPUTE_WARPS);
      mbar_init(&w_full[i], NUM_COMPUTE_WARPS);
      mbar_init(&w_empty[i], store_ds ? 2 : 1);
      mbar_init(&stats_full[i], NUM_COMPUTE_WARPS * 32);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_T1 = tmem_base;         // 2 x 64 columns
  const uint32_t tmem_T2 = tmem_base + 128;   // 2 x 64 columns
  const uint32_t tmem_A1 = tmem_base + 256;   // D columns
  const uint32_t tmem_A2 = tmem_base + 384;   // D columns (DKV only)

  if (warp == 0) {
    // -------------------------------------------------------------- TMA producer
    if (lane == 0 && n_iters > 0) {
      mbar_expect_tx(x_full, 2 * L::kX);
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        tma_load_4d(smem + L::kOffX1 + c * (BP * 128), &tmX1, x_full, c * 64, hp, p0, b);
        tma_load_4d(smem + L::kOffX2 + c * (BP * 128), &tmX2, x_full, c * 64, hp, p0, b);
      }
      bool ok = true;
      int st = 0;
      uint32_t ph = 0;
      for (int it = 0; it < n_iters && ok; ++it) {
        const int g = MODE == kModeDQ ? 0 : it / n_sub;
        const int sub = s_lo + (MODE == kModeDQ ? it : it % n_sub);
        const int hy = MODE == kModeDQ ? kvh : kvh * group + g;
        if (!mbar_wait(&y_empty[st], ph ^ 1, abort_flag, p.status, kErrWaitEmpty)) { ok = false; break; }
        uint8_t* sy = smem + L::kOffY + st * 2 * L::kY;
        mbar_expect_tx(&y_full[st], 2 * L::kY);
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          tma_load_4d(sy + c * (BS * 128), &tmY1, &y_full[st], c * 64, hy, sub * BS, b);
          tma_load_4d(sy + L::kY + c * (BS * 128), &tmY2, &y_full[st], c * 64, hy, sub * BS, b);
        }
        if (++st == YSTAGES) { st = 0; ph ^= 1; }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_iters > 0) {
      constexpr uint32_t idesc_t = make_idesc_bf16(BP, BS, false, false);
      constexpr uint32_t idesc_a = make_idesc_bf16(BP, D, false, true);
      const uint64_t x1_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffX1), 16, 1024);
      const uint64_t x2_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffX2), 16, 1024);
      const uint64_t y_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffY), 16, 1024);           // K-major view
      const uint64_t ymn_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffY), BS * 128, 1024);  // MN-major view
      const uint64_t w_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffW), 16, 1024);
      auto issue_t = [&](int it) -> bool {
        const int yst = it % YSTAGES;
        const uint32_t yph = (it / YSTAGES) & 1;
        const int tb = it & 1;
        const uint32_t tph = (it >> 1) & 1;
        if (!mbar_wait(&y_full[yst], yph, abort_flag, p.status, kErrWaitFull)) return false;
        if (!mbar_wait(&t_empty[tb], tph ^ 1, abort_flag, p.status, kErrWaitTmemEmpty)) return false;
        tc_fence_after();
        const uint64_t dy1 = y_desc0 + static_cast<uint64_t>(yst * ((2 * L::kY) >> 4));
        const uint64_t dy2 = dy1 + static_cast<uint64_t>(L::kY >> 4);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t xo = static_cast<uint64_t>(((k / 4) * (BP * 128) + (k % 4) * 32) >> 4);
          const uint64_t yo = static_cast<uint64_t>(((k / 4) * (BS * 128) + (k % 4) * 32) >> 4);
          mma_f16_ss(tmem_T1 + tb * BS, x1_desc0 + xo, dy1 + yo, idesc_t, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t xo = static_cast<uint64_t>(((k / 4) * (BP * 128) + (k % 4) * 32) >> 4);
          const uint64_t yo = static_cast<uint64_t>(((k / 4) * (BS * 128) + (k % 4) * 32) >> 4);
          mma_f16_ss(tmem_T2 + tb * BS, x2_desc0 + xo, dy2 + yo, idesc_t, k > 0 ? 1u : 0u);
        }
        mma_commit(&t_full[tb]);
        return true;
      };
      auto issue_acc = [&](int it) -> bool {
        const int yst = it % YSTAGES;
        const int tb = it & 1;
        const uint32_t tph = (it >> 1) & 1;
        if (!mbar_wait(&w_full[tb], tph, abort_flag, p.status, kErrWaitOther)) return false;
        tc_fence_after();
        if (store_ds) {
          const int g = it / n_sub;
          const int s0 = (s_lo + it % n_sub) * BS;
          tma_store_4d(&tmDS, smem + L::kOffW + tb * NW * L::kW, s0, p0, kvh * group + g, b);
          tma_store_commit();
        }
        const uint64_t dw = w_desc0 + static_cast<uint64_t>(tb * ((NW * L::kW) >> 4));
        const uint64_t dy1 = ymn_desc0 + static_cast<uint64_t>(yst * ((2 * L::kY) >> 4));
        const uint64_t dy2 = dy1 + static_cast<uint64_t>(L::kY >> 4);
#pragma unroll
        for (int k = 0; k < BS / 16; ++k) {
          // A: ds tile, K-major, one 64-wide chunk; B: Y1 re-read MN-major (64-row K extent)
          mma_f16_ss(tmem_A1, dw + static_cast<uint64_t>((k * 32) >> 4), dy1 + static_cast<uint64_t>((k * 16 * 128) >> 4),
                     idesc_a, (it > 0 || k > 0) ? 1u : 0u);
        }
        if (MODE == kModeDKV) {
#pragma unroll
          for (int k = 0; k < BS / 16; ++k) {
            if constexpr (P_IN_TMEM)
              mma_f16_ts(tmem_A2, tmem_T1 + tb * BS + k * 16, dy2 + static_cast<uint64_t>((k * 16 * 128) >> 4), idesc_a,
                         (it > 0 || k > 0) ? 1u : 0u);
            else
              mma_f16_ss(tmem_A2, dw + static_cast<uint64_t>((L::kW + k * 32) >> 4),
                         dy2 + static_cast<uint64_t>((k * 16 * 128) >> 4), idesc_a, (it > 0 || k > 0) ? 1u : 0u);
          }
        }
        mma_commit(&y_empty[yst]);
        mma_commit(&w_empty[tb]);
        return true;
      };
      bool ok = mbar_wait(x_full, 0, abort_flag, p.status, kErrWaitFull);
      if (ok) ok = issue_t(0);
      if (ok && n_iters > 1) ok = issue_t(1);
      for (int it = 0; it < n_iters && ok; ++it) {
        ok = issue_acc(it);
        if (ok && it + 2 < n_iters) ok = issue_t(it + 2);
        if (ok && store_ds) {
          tma_store_wait_read<0>();
          mbar_arrive(&w_empty[it & 1]);
        }
      }
      if (ok) mma_commit(acc_full);
      tma_store_wait<0>();
    }
  } else {
    // -------------------------------------------------------------- compute warps
    const int qd = warp & 3;
    const int row = qd * 32 + lane;  // primary row inside the tile
    const int tid128 = (warp - 2) * 32 + lane;  // index among the compute threads
    const int ch = (warp - 2) >> 2;              // which CW-column slice of the tile this warp takes
    const uint32_t lane_sel = static_cast<uint32_t>(qd * 32) << 16;
    const int prow = p0 + row;
    const float kLog2e = 1.4426950408889634f;
    float my_lse2 = 0.0f, my_delta = 0.0f;
    if (MODE == kModeDQ && prow < p.Tq) {
      const long long si = (static_cast<long long>(b) * p.H + hp) * p.Tq + prow;
      my_lse2 = p.lse[si] * kLog2e;
      my_delta = p.delta[si];
    }
    bool ok = true;
    // DKV mode: threads 0..63 carry lse (log2 units), threads 64..127 carry delta of query row s0 + (tid & 63)
    auto load_stat = [&](int it) -> float {
      const int g = it / n_sub;
      const int q = (s_lo + it % n_sub) * BS + (tid128 & (BS - 1));
      if (tid128 >= 2 * BS || q >= p.Tq) return 0.0f;
      const long long si = (static_cast<long long>(b) * p.H + (kvh * group + g)) * p.Tq + q;
      return tid128 < BS ? p.lse[si] * kLog2e : p.delta[si];
    };
    auto publish_stat = [&](int buf, float v) {
      float* base = stats + buf * 2 * BS;
      if (tid128 < 2 * BS) base[tid128] = v;  // [0,64) lse, [64,128) delta
      mbar_arrive(&stats_full[buf]);
    };
    if (MODE == kModeDKV && n_iters > 0) publish_stat(0, load_stat(0));
    for (int it = 0; it < n_iters && ok; ++it) {
      const int tb = it & 1;
      const uint32_t tph = (it >> 1) & 1;
      const int g = MODE == kModeDQ ? 0 : it / n_sub;
      const int sub = s_lo + (MODE == kModeDQ ? it : it % n_sub);
      const int s0 = sub * BS;  // first secondary row (key for DQ, query row for DKV)
      float* st_lse = stats + tb * 2 * BS;
      float* st_delta = st_lse + BS;
      float next_stat = 0.0f;
      if (MODE == kModeDKV) {
        // fetch the statistics of the NEXT sub-tile now; they are published at the end of this iteration,
        // so the global-load latency never sits on the critical path
        if (it + 1 < n_iters) next_stat = load_stat(it + 1);
        if (!mbar_wait(&stats_full[tb], tph, abort_flag, p.status, kErrWaitOther)) { ok = false; break; }
      }
      // does any element of this 128 x 64 block need masking?
      bool need_mask;
      if (MODE == kModeDQ) {
        const int qf = p.q_offset + p0, ql = p.q_offset + p0 + BP - 1;
        need_mask = (s0 + BS - 1 > qf) || (p.window_left >= 0 && s0 < ql - p.window_left) || (s0 + BS > p.Tk);
      } else {
        const int qf = p.q_offset + s0, ql = p.q_offset + s0 + BS - 1;
        need_mask = (p0 + BP - 1 > qf) || (p.window_left >= 0 && p0 < ql - p.window_left) || (s0 + BS > p.Tq) ||
                    (p0 + BP > p.Tk);
      }
      if (!mbar_wait(&t_full[tb], tph, abort_flag, p.status, kErrWaitTmemFull)) { ok = false; break; }
      tc_fence_after();
      if (!mbar_wait(&w_empty[tb], tph ^ 1, abort_flag, p.status, kErrWaitOther)) { ok = false; break; }
      uint8_t* sW = smem + L::kOffW + tb * NW * L::kW + row * 128;
      {
        const int c0 = ch * CW;  // first column of this warp
        uint32_t t1[CW], t2[CW];
        if constexpr (CW == 32) {
          tmem_ld_32x32(tmem_T1 + tb * BS + c0 + lane_sel, t1);
          tmem_ld_32x32(tmem_T2 + tb * BS + c0 + lane_sel, t2);
        } else {
          tmem_ld_32x16(tmem_T1 + tb * BS + c0 + lane_sel, t1);
          tmem_ld_32x16(tmem_T2 + tb * BS + c0 + lane_sel, t2);
        }
        tmem_ld_wait();
        uint32_t pk_ds[CW / 2], pk_p[CW / 2];
#pragma unroll
        for (int e = 0; e < CW; e += 2) {
          float pv[2], dsv[2];
          float lse_pair[2] = {0.0f, 0.0f}, delta_pair[2] = {0.0f, 0.0f};
          if (MODE == kModeDKV) {
            const float2 a = *reinterpret_cast<const float2*>(st_lse + c0 + e);
            const float2 d2 = *reinterpret_cast<const float2*>(st_delta + c0 + e);
            lse_pair[0] = a.x, lse_pair[1] = a.y, delta_pair[0] = d2.x, delta_pair[1] = d2.y;
          }
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int col = c0 + e + u;
            const float lse2 = MODE == kModeDQ ? my_lse2 : lse_pair[u];
            const float dl = MODE == kModeDQ ? my_delta : delta_pair[u];
            float pe = fast_exp2(__uint_as_float(t1[e + u]) * p.scale_log2 - lse2);
            if (need_mask) {
              const int key = MODE == kModeDQ ? s0 + col : prow;
              const int qrow = MODE == kModeDQ ? prow : s0 + col;
              const int qpos = p.q_offset + qrow;
              const bool allowed = key <= qpos && key < p.Tk && qrow < p.Tq &&
                                   (p.window_left < 0 || qpos - key <= p.window_left);
              pe = allowed ? pe : 0.0f;
            }
            pv[u] = pe;
            dsv[u] = pe * (__uint_as_float(t2[e + u]) - dl) * p.scale;
          }
          pk_ds[e / 2] = pack_bf16(dsv[0], dsv[1]);
          if (MODE == kModeDKV) pk_p[e / 2] = pack_bf16(pv[0], pv[1]);
        }
#pragma unroll
        for (int gq = 0; gq < CW / 8; ++gq) {
          const int gran = (ch * (CW / 8) + gq) ^ (row & 7);
          *reinterpret_cast<uint4*>(sW + gran * 16) =
              make_uint4(pk_ds[4 * gq], pk_ds[4 * gq + 1], pk_ds[4 * gq + 2], pk_ds[4 * gq + 3]);
          if (MODE == kModeDKV && !P_IN_TMEM)
            *reinterpret_cast<uint4*>(sW + L::kW + gran * 16) =
                make_uint4(pk_p[4 * gq], pk_p[4 * gq + 1], pk_p[4 * gq + 2], pk_p[4 * gq + 3]);
        }
        if constexpr (P_IN_TMEM) {
          tmem_st_32x8(tmem_T1 + tb * BS + c0 + lane_sel, pk_p);
          tmem_st_wait();
        }
      }
      tc_fence_before();
      fence_async_shared();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&t_empty[tb]);
        mbar_arrive(&w_full[tb]);
      }
      if (MODE == kModeDKV && it + 1 < n_iters) publish_stat(tb ^ 1, next_stat);
    }
    // ---- epilogue: accumulators -> bf16 -> global
    const bool have = n_iters > 0;
    if (ok && have) ok = mbar_wait(acc_full, 0, abort_flag, p.status, kErrWaitTmemFull);
    if (ok) {
      tc_fence_after();
      const int t_limit = MODE == kModeDQ ? p.Tq : p.Tk;
      const bool row_ok = prow < t_limit;
#pragma unroll
      for (int which = 0; which < NW; ++which) {
        __nv_bfloat16* base = which == 0 ? p.out1 : p.out2;
        const long long sb = which == 0 ? p.o1_stride_b : p.o2_stride_b;
        const long long stt = which == 0 ? p.o1_stride_t : p.o2_stride_t;
        const long long sh = which == 0 ? p.o1_stride_h : p.o2_stride_h;
        __nv_bfloat16* op = base + b * sb + static_cast<long long>(prow) * stt + static_cast<long long>(hp) * sh;
        const uint32_t tacc = which == 0 ? tmem_A1 : tmem_A2;
        // the warps of a quadrant split the D accumulator columns; chunks of EW columns
        constexpr int EC = D / (NUM_COMPUTE_WARPS / 4);
        constexpr int EW = EC >= 32 ? 32 : 16;
#pragma unroll 1
        for (int c = ch * EC; c < (ch + 1) * EC; c += EW) {
          uint32_t r[EW];
          if (have) {
            if constexpr (EW == 32) tmem_ld_32x32(tacc + c + lane_sel, r);
            else tmem_ld_32x16(tacc + c + lane_sel, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < EW; ++e) r[e] = 0u;
          }
          if (row_ok) {
#pragma unroll
            for (int gq = 0; gq < EW / 8; ++gq) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                w[e] = pack_bf16(__uint_as_float(r[gq * 8 + e * 2]), __uint_as_float(r[gq * 8 + e * 2 + 1]));
              *reinterpret_cast<uint4*>(op + c + gq * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]; one warp per (token, head)
__global__ void __launch_bounds__(256) attention_delta_kernel(const __nv_bfloat16* __restrict__ O, long long osb,
                                                              long long ost, long long osh,
                                                              const __nv_bfloat16* __restrict__ dO, long long dsb,
                                                              long long dst, long long dsh, float* __restrict__ delta,
                                                              int B, int H, int T, int D) {
  const long long wid = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (wid >= static_cast<long long>(B) * T * H) return;
  const int lane = threadIdx.x & 31;
  const int h = static_cast<int>(wid % H);
  const long long bt = wid / H;
  const int t = static_cast<int>(bt % T);
  const int b = static_cast<int>(bt / T);
  const __nv_bfloat16* op = O + b * osb + static_cast<long long>(t) * ost + static_cast<long long>(h) * osh;
  const __nv_bfloat16* dp = dO + b * dsb + static_cast<long long>(t) * dst + static_cast<long long>(h) * dsh;
  float acc = 0.0f;
  for (int d = lane * 2; d < D; d += 64) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(op + d);
    const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(dp + d);
    acc += __bfloat162float(a.x) * __bfloat162float(g.x) + __bfloat162float(a.y) * __bfloat162float(g.y);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) delta[(static_cast<long long>(b) * H + h) * T + t] = acc;
}

// The same sum with 16-byte loads: D / 8 lanes share a row, a warp covers 32 / (D / 8) rows per pass and keeps four
// passes (eight loads per thread) in flight, so the kernel runs at memory speed (it reads O and dO once).
template <int D>
__global__ void __launch_bounds__(256) attention_delta_vec_kernel(const __nv_bfloat16* __restrict__ O, long long osb,
                                                                  long long ost, long long osh,
                                                                  const __nv_bfloat16* __restrict__ dO, long long dsb,
                                                                  long long dst, long long dsh,
                                                                  float* __restrict__ delta, int B, int H, int T) {
  constexpr int LPR = D / 8;     // lanes per row
  constexpr int RPW = 32 / LPR;  // rows per warp and pass
  constexpr int UNROLL = 4;
  const int lane = threadIdx.x & 31, sub = lane / LPR, li = lane % LPR;
  const long long n = static_cast<long long>(B) * T * H;
  const long long warp_global = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const long long step = static_cast<long long>(gridDim.x) * 8 * RPW * UNROLL;
  for (long long base = warp_global * RPW * UNROLL; base < n; base += step) {
    uint4 a[UNROLL], g[UNROLL];
    long long out[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long r = base + u * RPW + sub;
      out[u] = -1;
      a[u] = g[u] = make_uint4(0, 0, 0, 0);
      if (r < n) {
        const int h = static_cast<int>(r % H);
        const long long bt = r / H;
        const int t = static_cast<int>(bt % T);
        const long long b = bt / T;
        a[u] = *reinterpret_cast<const uint4*>(O + b * osb + static_cast<long long>(t) * ost +
                                               static_cast<long long>(h) * osh + li * 8);
        g[u] = *reinterpret_cast<const uint4*>(dO + b * dsb + static_cast<long long>(t) * dst +
                                               static_cast<long long>(h) * dsh + li * 8);
        out[u] = (b * H + h) * T + t;
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const uint32_t aw[4] = {a[u].x, a[u].y, a[u].z, a[u].w}, gw[4] = {g[u].x, g[u].y, g[u].z, g[u].w};
      float acc = 0.0f;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        acc += __uint_as_float(aw[e] << 16) * __uint_as_float(gw[e] << 16) +
               __uint_as_float(aw[e] & 0xffff0000u) * __uint_as_float(gw[e] & 0xffff0000u);
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (li == 0 && out[u] >= 0) delta[out[u]] = acc;
    }
  }
}

template <int D, int MODE>
const char* launch_bwd(const CUtensorMap& x1, const CUtensorMap& x2, const CUtensorMap& y1, const CUtensorMap& y2,
                       const CUtensorMap& ds, const BwdParams& p, dim3 grid, cudaStream_t stream) {
  using L = BwdSmem<D, MODE>;
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(attention_bwd_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         L::kTotal);
    if (e != cudaSuccess) return cudaGetErrorString(e);
    cfg = true;
  }
  attention_bwd_kernel<D, MODE><<<grid, BwdWarps<MODE>::kThreads, L::kTotal, stream>>>(x1, x2, y1, y2, ds, p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace

const char* attention_bwd(const AttnArgs& a, cudaStream_t stream) {
  if (a.D != 64 && a.D != 128) return "attention_bwd: head_dim must be 64 or 128";
  if (a.H % a.KVH) return "attention_bwd: heads must be a multiple of kv heads";
  {
    const long long n = static_cast<long long>(a.B) * a.Tq * a.H;
    const __nv_bfloat16* o = static_cast<const __nv_bfloat16*>(a.O);
    const __nv_bfloat16* g = static_cast<const __nv_bfloat16*>(a.dO);
    auto mult8 = [](long long v) { return v % 8 == 0; };
    const bool vec = ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(g)) & 15) == 0 &&
                     mult8(a.o_stride_b) && mult8(a.o_stride_t) && mult8(a.o_stride_h) && mult8(a.do_stride_b) &&
                     mult8(a.do_stride_t) && mult8(a.do_stride_h);
    const long long rows_per_cta = 8 * (32 / (a.D / 8)) * 4;
    const unsigned ctas = static_cast<unsigned>(std::min<long long>((n + rows_per_cta - 1) / rows_per_cta, 148 * 16));
    if (vec && a.D == 128)
      attention_delta_vec_kernel<128><<<ctas, 256, 0, stream>>>(o, a.o_stride_b, a.o_stride_t, a.o_stride_h, g,
                                                                 a.do_stride_b, a.do_stride_t, a.do_stride_h, a.delta,
                                                                 a.B, a.H, a.Tq);
    else if (vec && a.D == 64)
      attention_delta_vec_kernel<64><<<ctas, 256, 0, stream>>>(o, a.o_stride_b, a.o_stride_t, a.o_stride_h, g,
                                                                a.do_stride_b, a.do_stride_t, a.do_stride_h, a.delta, a.B,
                                                                a.H, a.Tq);
    else
      attention_delta_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, stream>>>(
          o, a.o_stride_b, a.o_stride_t, a.o_stride_h, g, a.do_stride_b, a.do_stride_t, a.do_stride_h, a.delta, a.B,
          a.H, a.Tq, a.D);
  }
  CUtensorMap q128, do128, k128, v128, q64, do64, k64, v64;
  const long long dq[4] = {a.D, a.H, a.Tq, a.B};
  const long long dk[4] = {a.D, a.KVH, a.Tk, a.B};
  const long long sq[3] = {a.q_stride_h, a.q_stride_t, a.q_stride_b};
  const long long sdo[3] = {a.do_stride_h, a.do_stride_t, a.do_stride_b};
  const long long sk[3] = {a.k_stride_h, a.k_stride_t, a.k_stride_b};
  const long long sv[3] = {a.v_stride_h, a.v_stride_t, a.v_stride_b};
  const int box128[4] = {64, 1, BP, 1};
  const int box64[4] = {64, 1, BS, 1};
  bool ok = make_tmap_bf16_4d(&q128, a.Q, dq, sq, box128) && make_tmap_bf16_4d(&do128, a.dO, dq, sdo, box128) &&
            make_tmap_bf16_4d(&k128, a.K, dk, sk, box128) && make_tmap_bf16_4d(&v128, a.V, dk, sv, box128) &&
            make_tmap_bf16_4d(&q64, a.Q, dq, sq, box64) && make_tmap_bf16_4d(&do64, a.dO, dq, sdo, box64) &&
            make_tmap_bf16_4d(&k64, a.K, dk, sk, box64) && make_tmap_bf16_4d(&v64, a.V, dk, sv, box64);
  if (!ok) return "attention_bwd: tensor map construction failed";
  BwdParams p;
  p.B = a.B, p.H = a.H, p.KVH = a.KVH, p.Tq = a.Tq, p.Tk = a.Tk;
  p.q_offset = a.q_offset, p.window_left = a.window_left;
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.lse = a.lse;
  p.delta = a.delta;
  p.status = a.status;
  p.ds_out = static_cast<__nv_bfloat16*>(a.dS);
  p.ds_tk = a.ds_tk, p.ds_tq = a.ds_tq;
  if (a.dS != nullptr && (a.ds_tk < (a.Tk + 127) / 128 * 128 || a.ds_tq < (a.Tq + 127) / 128 * 128 || a.ds_tq % 8))
    return "attention_bwd: dS scratch is too small";
  CUtensorMap ds_map = q64;  // placeholder when there is no scratch (never dereferenced then)
  if (a.dS != nullptr) {
    const long long dd[4] = {a.ds_tq, a.ds_tk, a.H, a.B};
    const long long sd[3] = {a.ds_tq, a.ds_tq * a.ds_tk, a.ds_tq * a.ds_tk * a.H};
    const int boxd[4] = {BS, BP, 1, 1};
    if (!make_tmap_bf16_4d(&ds_map, a.dS, dd, sd, boxd)) return "attention_bwd: dS tensor map construction failed";
  }
  const char* err;
  // dK, dV
  p.out1 = static_cast<__nv_bfloat16*>(a.dK);
  p.o1_stride_b = a.dk_stride_b, p.o1_stride_t = a.dk_stride_t, p.o1_stride_h = a.dk_stride_h;
  p.out2 = static_cast<__nv_bfloat16*>(a.dV);
  p.o2_stride_b = a.dv_stride_b, p.o2_stride_t = a.dv_stride_t, p.o2_stride_h = a.dv_stride_h;
  const dim3 grid_kv((a.Tk + BP - 1) / BP, a.KVH, a.B);
  err = a.D == 128 ? launch_bwd<128, kModeDKV>(k128, v128, q64, do64, ds_map, p, grid_kv, stream)
                   : launch_bwd<64, kModeDKV>(k128, v128, q64, do64, ds_map, p, grid_kv, stream);
  if (err) return err;
  if (a.dS != nullptr) return attention_dq_from_ds(a, stream);
  // dQ
  p.ds_out = nullptr;
  p.out1 = static_cast<__nv_bfloat16*>(a.dQ);
  p.o1_stride_b = a.dq_stride_b, p.o1_stride_t = a.dq_stride_t, p.o1_stride_h = a.dq_stride_h;
  p.out2 = nullptr;
  const dim3 grid_q((a.Tq + BP - 1) / BP, a.H, a.B);
  err = a.D == 128 ? launch_bwd<128, kModeDQ>(q128, do128, k64, v64, ds_map, p, grid_q, stream)
                   : launch_bwd<64, kModeDQ>(q128, do128, k64, v64, ds_map, p, grid_q, stream);
  return err;
}

}  // namespace nc

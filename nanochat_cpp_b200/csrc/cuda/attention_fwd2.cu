// Sliding-window GQA flash attention, forward, two query tiles per CTA (sm_100a).
//
// One CTA per (256 query rows, head, batch), 320 threads:
//   warp 0        TMA producer: both Q tiles once, then 3-stage rings of 64-key K and V tiles
//   warp 1        tcgen05.mma issuer for both query tiles: S^x_j = Q^x K_j^T (two TMEM score buffers per
//                 tile) and O^x += P^x_j V_j, with O accumulating in TMEM across the whole key sweep
//   warps 2..5    softmax of query tile 0   } each thread owns one query row; exp2 with folded scale;
//   warps 6..9    softmax of query tile 1   } P goes to shared memory (128-byte swizzle, K-major)
// The running maximum is only raised when a tile exceeds it by more than 2^8 in the exponent domain;
// then (rarely: the first tiles of a row) the thread rescales its O row in TMEM. Otherwise probabilities
// are taken against the stale maximum, which is exact after the final division by the row sum. With
// two softmax warpgroups the tensor core and the exponential unit overlap across the two tiles.
// Key visibility and statistics are those of attention_fwd.cu (reference backends/cpu/kernels.cc:879-964).
#include <cuda.h>
#include <cuda_bf16.h>
#include <math_constants.h>

#include "attention.h"
#include "ptx.cuh"
#include "tmap.h"

namespace nc {

namespace {

constexpr int BQ = 128;    // rows per query tile (TMEM lanes)
constexpr int NQ = 2;      // query tiles per CTA
constexpr int BKV = 64;    // keys per step
constexpr int KVSTAGES = 3;
constexpr int NUM_THREADS = 64 + NQ * 128;
constexpr float kRescaleThreshold = 8.0f;  // in log2 units
// The probabilities stay in tensor memory: each thread packs its row of P to bf16 and stores it over the first 32
// of the 64 score columns it has just read; the P V product takes its A operand from there. The score buffer is
// next written by the score MMA two key tiles later, which the MMA thread issues after this tile's P V product,
// and MMAs run in issue order, so no extra barrier is needed. Shared memory carries only Q, K and V.
constexpr bool kPInTmem = true;

template <int D>
struct Fwd2Smem {
  static constexpr int kQ = BQ * D * 2;
  static constexpr int kKV = BKV * D * 2;
  static constexpr int kP = BQ * BKV * 2;
  static constexpr int kOffQ = 0;                               // NQ tiles
  static constexpr int kOffK = kOffQ + NQ * kQ;                 // KVSTAGES
  static constexpr int kOffV = kOffK + KVSTAGES * kKV;          // KVSTAGES
  static constexpr int kOffP = kOffV + KVSTAGES * kKV;          // NQ x 2 buffers
  static constexpr int kOffBar = kOffP + NQ * 2 * kP;
  static constexpr int kTotal = kOffBar + 512 + 1024;
};

struct Fwd2Params {
  int B, H, KVH, Tq, Tk;
  int q_offset, window_left;
  float scale_log2;
  __nv_bfloat16* O;
  long long o_stride_b, o_stride_t, o_stride_h;
  float* lse;
  int* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// key-tile range [lo, hi] (64-key tiles) visible to query rows [q0, q0 + BQ)
__device__ __forceinline__ void tile_range(const Fwd2Params& p, int q0, int& lo, int& hi) {
  if (q0 >= p.Tq) {
    lo = 0;
    hi = -1;
    return;
  }
  const int q_first = p.q_offset + q0;
  const int q_last = p.q_offset + min(q0 + BQ - 1, p.Tq - 1);
  const int first_key = p.window_left >= 0 ? max(0, q_first - p.window_left) : 0;
  lo = first_key / BKV;
  hi = min(q_last, p.Tk - 1) / BKV;
}

template <int D>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attention_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const Fwd2Params p) {
  using L = Fwd2Smem<D>;
  constexpr int DC = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [3]
  uint64_t* k_empty = bars + 4;   // [3]
  uint64_t* v_full = bars + 7;    // [3]
  uint64_t* v_empty = bars + 10;  // [3]
  // per query tile x: 10 barriers starting at bars + 13 + 10x
  auto s_full = [&](int x, int i) { return bars + 13 + 10 * x + i; };
  auto s_empty = [&](int x, int i) { return bars + 15 + 10 * x + i; };
  auto p_full = [&](int x, int i) { return bars + 17 + 10 * x + i; };
  auto p_empty = [&](int x, int i) { return bars + 19 + 10 * x + i; };
  // o_done flips after every P V product of the tile (the rescale path waits on it by parity: at step i the scores
  // of tile i are already in hand, so at least i - 1 products are complete and the parity is unambiguous).
  // o_final completes once, after the LAST product: the epilogue cannot use o_done, because a thread that has
  // finished the last tile's probabilities only knows that n - 2 products are complete, and a parity wait cannot
  // tell n - 2 completions from n.
  auto o_done = [&](int x) { return bars + 21 + 10 * x; };
  auto o_final = [&](int x) { return bars + 22 + 10 * x; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13 + 10 * NQ);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q_blocks = (p.Tq + NQ * BQ - 1) / (NQ * BQ);
  const int q_block = q_blocks - 1 - blockIdx.x;  // heaviest first
  const int q_base = q_block * NQ * BQ;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int kvh = h / (p.H / p.KVH);
  int lo[NQ], hi[NQ];
#pragma unroll
  for (int x = 0; x < NQ; ++x) tile_range(p, q_base + x * BQ, lo[x], hi[x]);
  // union range (tile 0 always exists; tile 1 may be empty)
  const int lo_u = (hi[1] >= lo[1]) ? min(lo[0], lo[1]) : lo[0];
  const int hi_u = max(hi[0], hi[1]);
  const int n_u = hi_u - lo_u + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < KVSTAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int x = 0; x < NQ; ++x) {
      for (int i = 0; i < 2; ++i) {
        mbar_init(s_full(x, i), 1);
        mbar_init(s_empty(x, i), 4);
        mbar_init(p_full(x, i), 4);
        mbar_init(p_empty(x, i), 1);
      }
      mbar_init(o_done(x), 1);
      mbar_init(o_final(x), 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // S^x: 2 x 64 columns at x*128; O^x: D columns at 256 + x*128
  auto tmem_S = [&](int x, int buf) { return tmem_base + x * 128 + buf * BKV; };
  auto tmem_O = [&](int x) { return tmem_base + 256 + x * 128; };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, NQ * L::kQ);
#pragma unroll
      for (int x = 0; x < NQ; ++x)
#pragma unroll
        for (int c = 0; c < DC; ++c)
          tma_load_4d(smem + L::kOffQ + x * L::kQ + c * (BQ * 128), &tmQ, q_full, c * 64, h, q_base + x * BQ, b);
      bool ok = true;
      int st = 0;
      uint32_t ph = 0;
      for (int s = 0; s < n_u && ok; ++s) {
        const int kv0 = (lo_u + s) * BKV;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, kErrWaitEmpty)) { ok = false; break; }
        mbar_expect_tx(&k_full[st], L::kKV);
#pragma unroll
        for (int c = 0; c < DC; ++c)
          tma_load_4d(smem + L::kOffK + st * L::kKV + c * (BKV * 128), &tmK, &k_full[st], c * 64, kvh, kv0, b);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, kErrWaitEmpty)) { ok = false; break; }
        mbar_expect_tx(&v_full[st], L::kKV);
#pragma unroll
        for (int c = 0; c < DC; ++c)
          tma_load_4d(smem + L::kOffV + st * L::kKV + c * (BKV * 128), &tmV, &v_full[st], c * 64, kvh, kv0, b);
        if (++st == KVSTAGES) { st = 0; ph ^= 1; }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BQ, BKV, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(BQ, D, false, true);
      const uint64_t q_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffQ), 16, 1024);
      const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffK), 16, 1024);
      const uint64_t p_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffP), 16, 1024);
      const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffV), BKV * 128, 1024);
      auto issue_s = [&](int s) -> bool {  // scores of key tile lo_u + s for every active query tile
        const int j = lo_u + s;
        const int st = s % KVSTAGES;
        const uint32_t ph = (s / KVSTAGES) & 1;
        if (!mbar_wait(&k_full[st], ph, abort_flag, p.status, kErrWaitFull)) return false;
        const uint64_t dk = k_desc0 + static_cast<uint64_t>(st * (L::kKV >> 4));
#pragma unroll
        for (int x = 0; x < NQ; ++x) {
          if (j < lo[x] || j > hi[x]) continue;
          const int i = j - lo[x];
          if (!mbar_wait(s_empty(x, i & 1), ((i >> 1) & 1) ^ 1, abort_flag, p.status, kErrWaitTmemEmpty)) return false;
          tc_fence_after();
          const uint64_t dq = q_desc0 + static_cast<uint64_t>(x * (L::kQ >> 4));
          const uint32_t ts = tmem_S(x, i & 1);
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint64_t qo = static_cast<uint64_t>(((k / 4) * (BQ * 128) + (k % 4) * 32) >> 4);
            const uint64_t ko = static_cast<uint64_t>(((k / 4) * (BKV * 128) + (k % 4) * 32) >> 4);
            mma_f16_ss(ts, dq + qo, dk + ko, idesc_s, k > 0 ? 1u : 0u);
          }
          mma_commit(s_full(x, i & 1));
        }
        mma_commit(&k_empty[st]);
        return true;
      };
      auto issue_o = [&](int s) -> bool {
        const int j = lo_u + s;
        const int st = s % KVSTAGES;
        const uint32_t ph = (s / KVSTAGES) & 1;
        if (!mbar_wait(&v_full[st], ph, abort_flag, p.status, kErrWaitFull)) return false;
        const uint64_t dv = v_desc0 + static_cast<uint64_t>(st * (L::kKV >> 4));
#pragma unroll
        for (int x = 0; x < NQ; ++x) {
          if (j < lo[x] || j > hi[x]) continue;
          const int i = j - lo[x];
          if (!mbar_wait(p_full(x, i & 1), (i >> 1) & 1, abort_flag, p.status, kErrWaitOther)) return false;
          tc_fence_after();
          const uint64_t dp = p_desc0 + static_cast<uint64_t>((x * 2 + (i & 1)) * (L::kP >> 4));
          const uint32_t to = tmem_O(x);
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k) {
            if constexpr (kPInTmem)
              mma_f16_ts(to, tmem_S(x, i & 1) + k * 8, dv + static_cast<uint64_t>((k * 16 * 128) >> 4), idesc_o,
                         (i > 0 || k > 0) ? 1u : 0u);
            else
              mma_f16_ss(to, dp + static_cast<uint64_t>((k * 32) >> 4), dv + static_cast<uint64_t>((k * 16 * 128) >> 4),
                         idesc_o, (i > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit(p_empty(x, i & 1));
          mma_commit(o_done(x));
          if (j == hi[x]) mma_commit(o_final(x));
        }
        mma_commit(&v_empty[st]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kErrWaitFull);
      for (int s = 0; s <= n_u && ok; ++s) {
        if (s < n_u) ok = issue_s(s);
        if (ok && s >= 1) ok = issue_o(s - 1);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warpgroups
    const int x = (warp - 2) >> 2;  // query tile of this warpgroup
    const int qd = warp & 3;        // TMEM lane quadrant
    const int row = qd * 32 + lane;
    const int q0 = q_base + x * BQ;
    const int qpos = p.q_offset + q0 + row;
    const bool row_ok = (q0 + row) < p.Tq;
    const uint32_t lane_sel = static_cast<uint32_t>(qd * 32) << 16;
    const int n_x = hi[x] - lo[x] + 1;
    float m_ref = -1.0e30f, l_run = 0.0f;
    bool ok = true;
    for (int i = 0; i < n_x && ok; ++i) {
      const int sb = i & 1;
      const uint32_t ph = (i >> 1) & 1;
      const int kv0 = (lo[x] + i) * BKV;
      const bool need_mask = (kv0 + BKV - 1 > p.q_offset + q0) ||
                             (p.window_left >= 0 && kv0 < p.q_offset + q0 + BQ - 1 - p.window_left) ||
                             (kv0 + BKV > p.Tk);
      if (!mbar_wait(s_full(x, sb), ph, abort_flag, p.status, kErrWaitTmemFull)) { ok = false; break; }
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld_32x32(tmem_S(x, sb) + lane_sel, r0);
      tmem_ld_32x32(tmem_S(x, sb) + 32 + lane_sel, r1);
      tmem_ld_wait();
      // the scores are in registers: the MMA warp may overwrite this buffer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty(x, sb));
      float sv[64];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        sv[e] = __uint_as_float(r0[e]);
        sv[32 + e] = __uint_as_float(r1[e]);
      }
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < 64; ++e) {
          const int key = kv0 + e;
          const bool allowed = key <= qpos && key < p.Tk && (p.window_left < 0 || qpos - key <= p.window_left);
          sv[e] = allowed ? sv[e] : -CUDART_INF_F;  // exp2(-inf - m) is exactly 0 whatever the reference maximum
        }
      }
      float m_tile = -1.0e30f;
#pragma unroll
      for (int e = 0; e < 64; ++e) m_tile = fmaxf(m_tile, sv[e]);
      // raise the reference maximum only when the tile exceeds it by more than the threshold
      const bool raise = (m_tile - m_ref) * p.scale_log2 > kRescaleThreshold;
      if (__any_sync(0xffffffffu, raise)) {
        float alpha = 1.0f;
        if (raise) {
          alpha = fast_exp2((m_ref - m_tile) * p.scale_log2);
          m_ref = m_tile;
          l_run *= alpha;
        }
        if (i > 0) {
          // O^x must be quiescent: every product issued so far for this tile has to be complete
          if (!mbar_wait(o_done(x), (i - 1) & 1, abort_flag, p.status, kErrWaitTmemFull)) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < D / 16; ++c) {
            uint32_t o[16];
            tmem_ld_32x16(tmem_O(x) + c * 16 + lane_sel, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_32x16(tmem_O(x) + c * 16 + lane_sel, o);
          }
          tmem_st_wait();
          tc_fence_before();
        }
      }
      const float m_scaled = m_ref * p.scale_log2;
      uint32_t packed[32];
      float l_tile = 0.0f;
#pragma unroll
      for (int e = 0; e < 64; e += 2) {
        const float p0 = fast_exp2(sv[e] * p.scale_log2 - m_scaled);
        const float p1 = fast_exp2(sv[e + 1] * p.scale_log2 - m_scaled);
        const uint32_t pk = pack_bf16(p0, p1);
        l_tile += bf16_lo(pk) + bf16_hi(pk);
        packed[e / 2] = pk;
      }
      l_run += l_tile;
      if constexpr (kPInTmem) {
        tmem_st_32x32(tmem_S(x, sb) + lane_sel, packed);
        tmem_st_wait();
        tc_fence_before();
      } else {
        if (!mbar_wait(p_empty(x, sb), ph ^ 1, abort_flag, p.status, kErrWaitOther)) { ok = false; break; }
        uint8_t* sP = smem + L::kOffP + (x * 2 + sb) * L::kP + row * 128;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const int gran = g ^ (row & 7);
          *reinterpret_cast<uint4*>(sP + gran * 16) =
              make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
        }
        fence_async_shared();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(x, sb));
    }
    if (ok && n_x > 0) {
      if (mbar_wait(o_final(x), 0, abort_flag, p.status, kErrWaitTmemFull)) {
        tc_fence_after();
        const float inv_l = 1.0f / l_run;
        __nv_bfloat16* op = p.O + static_cast<long long>(b) * p.o_stride_b +
                            static_cast<long long>(q0 + row) * p.o_stride_t + static_cast<long long>(h) * p.o_stride_h;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_O(x) + c * 32 + lane_sel, r);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                w[e] = pack_bf16(__uint_as_float(r[g * 8 + e * 2]) * inv_l, __uint_as_float(r[g * 8 + e * 2 + 1]) * inv_l);
              *reinterpret_cast<uint4*>(op + c * 32 + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        if (row_ok)
          p.lse[(static_cast<long long>(b) * p.H + h) * p.Tq + q0 + row] =
              m_ref * p.scale_log2 * 0.6931471805599453f + logf(l_run);
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

}  // namespace

const char* attention_fwd2(const AttnArgs& a, cudaStream_t stream) {
  if (a.D != 64 && a.D != 128) return "attention_fwd: head_dim must be 64 or 128";
  if (a.H % a.KVH) return "attention_fwd: heads must be a multiple of kv heads";
  CUtensorMap tq, tk, tv;
  const long long dq[4] = {a.D, a.H, a.Tq, a.B};
  const long long sq[3] = {a.q_stride_h, a.q_stride_t, a.q_stride_b};
  const int boxq[4] = {64, 1, BQ, 1};
  const long long dk[4] = {a.D, a.KVH, a.Tk, a.B};
  const long long sk[3] = {a.k_stride_h, a.k_stride_t, a.k_stride_b};
  const long long sv[3] = {a.v_stride_h, a.v_stride_t, a.v_stride_b};
  const int boxk[4] = {64, 1, BKV, 1};
  if (!make_tmap_bf16_4d(&tq, a.Q, dq, sq, boxq) || !make_tmap_bf16_4d(&tk, a.K, dk, sk, boxk) ||
      !make_tmap_bf16_4d(&tv, a.V, dk, sv, boxk))
    return "attention_fwd: tensor map construction failed";
  Fwd2Params p;
  p.B = a.B, p.H = a.H, p.KVH = a.KVH, p.Tq = a.Tq, p.Tk = a.Tk;
  p.q_offset = a.q_offset, p.window_left = a.window_left;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.O = static_cast<__nv_bfloat16*>(a.O);
  p.o_stride_b = a.o_stride_b, p.o_stride_t = a.o_stride_t, p.o_stride_h = a.o_stride_h;
  p.lse = a.lse;
  p.status = a.status;
  const dim3 grid((a.Tq + NQ * BQ - 1) / (NQ * BQ), a.H, a.B);
  cudaError_t e;
  if (a.D == 128) {
    static bool cfg = false;
    if (!cfg) {
      e = cudaFuncSetAttribute(attention_fwd2_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               Fwd2Smem<128>::kTotal);
      if (e != cudaSuccess) return cudaGetErrorString(e);
      cfg = true;
    }
    attention_fwd2_kernel<128><<<grid, NUM_THREADS, Fwd2Smem<128>::kTotal, stream>>>(tq, tk, tv, p);
  } else {
    static bool cfg = false;
    if (!cfg) {
      e = cudaFuncSetAttribute(attention_fwd2_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               Fwd2Smem<64>::kTotal);
      if (e != cudaSuccess) return cudaGetErrorString(e);
      cfg = true;
    }
    attention_fwd2_kernel<64><<<grid, NUM_THREADS, Fwd2Smem<64>::kTotal, stream>>>(tq, tk, tv, p);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nc

// Sliding-window GQA flash attention, forward, for sm_100a.
//
// One CTA per (query tile of 128 rows, head, batch). 192 threads:
//   warp 0      TMA producer: Q once, then a 2-stage ring of K tiles and a 2-stage ring of V tiles
//   warp 1      tcgen05.mma issuer: S_j = Q K_j^T into one of two TMEM score buffers, then
//               O_j = P_j V_j into one of two TMEM output buffers (P_j comes from shared memory)
//   warps 2..5  softmax: each thread owns one query row (tcgen05.ld 32x32b hands a thread its row),
//               so row max / row sum need no shuffles; exp2 with the scale folded in; P_j is written
//               to shared memory in the 128-byte-swizzled K-major layout the MMA reads; the running
//               output is kept in registers and rescaled as new tiles arrive (O_{j-1} is folded in
//               after P_j has been published, so the tensor core never waits for the accumulate).
// Tiles outside the causal / left-window band are never loaded; only tiles that cross a band edge
// pay for masking. K and V tiles are fetched by TMA straight from the [B, T, H, D] activations (4-D
// tensor maps), so no head transpose pass exists.
//
// Semantics follow the reference CPU attention (backends/cpu/kernels.cc:879-964): key j is visible
// to query position q iff j <= q and (window_left < 0 or q - j <= window_left); GQA groups are
// contiguous; the saved statistic is lse = max + log(sum exp) per (batch, head, row).
#include "attention.h"

#include <cuda.h>
#include <cuda_bf16.h>

#include "ptx.cuh"
#include "tmap.h"

namespace nc {

namespace {

constexpr int BQ = 128;   // query rows per CTA
constexpr int BKV = 128;  // keys per tile
constexpr int NUM_THREADS = 192;

template <int D>
struct FwdSmem {
  static constexpr int kQ = BQ * D * 2;
  static constexpr int kKV = BKV * D * 2;
  static constexpr int kP = BQ * BKV * 2;
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kOffQ + kQ;       // 2 stages
  static constexpr int kOffV = kOffK + 2 * kKV;  // 2 stages
  static constexpr int kOffP = kOffV + 2 * kKV;  // 2 buffers
  static constexpr int kOffBar = kOffP + 2 * kP;
  static constexpr int kTotal = kOffBar + 256 + 1024;  // barriers + alignment slack
};

struct FwdParams {
  int B, H, KVH, Tq, Tk;
  int q_offset;     // absolute position of query row 0 (Tk - Tq for training)
  int window_left;  // < 0: full context
  float scale_log2; // softmax scale * log2(e)
  __nv_bfloat16* O;
  long long o_stride_b, o_stride_t, o_stride_h;
  float* lse;  // [B, H, Tq]
  int* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void kv_tile_range(const FwdParams& p, int q0, int& j_lo, int& j_hi) {
  const int q_first = p.q_offset + q0;
  const int q_last = min(p.q_offset + q0 + BQ - 1, p.q_offset + p.Tq - 1);
  int lo = 0;
  if (p.window_left >= 0) lo = max(0, q_first - p.window_left);
  j_lo = lo / BKV;
  j_hi = min(q_last, p.Tk - 1) / BKV;
}

template <int D>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  using L = FwdSmem<D>;
  constexpr int DC = D / 64;  // 64-element chunks of the head dimension
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* k_empty = bars + 3;  // [2]
  uint64_t* v_full = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;  // [2]
  uint64_t* s_full = bars + 9;   // [2]
  uint64_t* s_empty = bars + 11; // [2]
  uint64_t* p_full = bars + 13;  // [2]
  uint64_t* p_empty = bars + 15; // [2]
  uint64_t* o_full = bars + 17;  // [2]
  uint64_t* o_empty = bars + 19; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heaviest tiles (largest q0) first: blockIdx.x = 0 is the last query tile
  const int q_tiles = (p.Tq + BQ - 1) / BQ;
  const int q_tile = q_tiles - 1 - blockIdx.x;
  const int q0 = q_tile * BQ;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int kvh = h / (p.H / p.KVH);
  int j_lo, j_hi;
  kv_tile_range(p, q0, j_lo, j_hi);
  const int n_tiles = j_hi - j_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
      mbar_init(&p_full[i], 4);
      mbar_init(&p_empty[i], 1);
      mbar_init(&o_full[i], 1);
      mbar_init(&o_empty[i], 4);
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
  const uint32_t tmem_S = tmem_base;        // 2 x 128 columns
  const uint32_t tmem_O = tmem_base + 256;  // 2 x D columns

  if (warp == 0) {
    // -------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, L::kQ);
#pragma unroll
      for (int c = 0; c < DC; ++c) tma_load_4d(smem + L::kOffQ + c * (BQ * 128), &tmQ, q_full, c * 64, h, q0, b);
      bool ok = true;
      for (int it = 0; it < n_tiles && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int kv0 = (j_lo + it) * BKV;
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
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BQ, BKV, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(BQ, D, false, true);
      const uint64_t q_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffQ), 16, 1024);
      const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffK), 16, 1024);
      const uint64_t p_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffP), 16, 1024);
      const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(smem + L::kOffV), BKV * 128, 1024);
      auto issue_s = [&](int it) -> bool {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, abort_flag, p.status, kErrWaitFull)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, abort_flag, p.status, kErrWaitTmemEmpty)) return false;
        tc_fence_after();
        const uint64_t dk = k_desc0 + static_cast<uint64_t>(st * (L::kKV >> 4));
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t off = static_cast<uint64_t>(((k / 4) * (128 * 128) + (k % 4) * 32) >> 4);
          mma_f16_ss(tmem_S + st * 128, q_desc0 + off, dk + off, idesc_s, k > 0 ? 1u : 0u);
        }
        mma_commit(&k_empty[st]);
        mma_commit(&s_full[st]);
        return true;
      };
      auto issue_o = [&](int it) -> bool {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&v_full[st], ph, abort_flag, p.status, kErrWaitFull)) return false;
        if (!mbar_wait(&p_full[st], ph, abort_flag, p.status, kErrWaitOther)) return false;
        if (!mbar_wait(&o_empty[st], ph ^ 1, abort_flag, p.status, kErrWaitTmemEmpty)) return false;
        tc_fence_after();
        const uint64_t dp = p_desc0 + static_cast<uint64_t>(st * (L::kP >> 4));
        const uint64_t dv = v_desc0 + static_cast<uint64_t>(st * (L::kKV >> 4));
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint64_t a_off = static_cast<uint64_t>(((k / 4) * (BQ * 128) + (k % 4) * 32) >> 4);
          const uint64_t b_off = static_cast<uint64_t>((k * (16 * 128)) >> 4);
          mma_f16_ss(tmem_O + st * D, dp + a_off, dv + b_off, idesc_o, k > 0 ? 1u : 0u);
        }
        mma_commit(&v_empty[st]);
        mma_commit(&p_empty[st]);
        mma_commit(&o_full[st]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kErrWaitFull);
      if (ok) ok = issue_s(0);
      if (ok && n_tiles > 1) ok = issue_s(1);
      for (int it = 0; it < n_tiles && ok; ++it) {
        ok = issue_o(it);
        if (ok && it + 2 < n_tiles) ok = issue_s(it + 2);
      }
    }
  } else {
    // -------------------------------------------------------------- softmax + output accumulate
    const int qd = warp & 3;
    const int row = qd * 32 + lane;               // row inside the query tile
    const int qpos = p.q_offset + q0 + row;       // absolute position
    const bool row_ok = (q0 + row) < p.Tq;
    const uint32_t lane_sel = static_cast<uint32_t>(qd * 32) << 16;
    float o_acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o_acc[i] = 0.0f;
    float m_run = -1.0e30f, l_run = 0.0f, alpha_prev = 1.0f;
    bool ok = true;
    for (int it = 0; it < n_tiles && ok; ++it) {
      const int st = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const int kv0 = (j_lo + it) * BKV;
      const bool need_mask = (kv0 + BKV - 1 > p.q_offset + q0) ||
                             (p.window_left >= 0 && kv0 < p.q_offset + q0 + BQ - 1 - p.window_left) ||
                             (kv0 + BKV > p.Tk);
      if (!mbar_wait(&s_full[st], ph, abort_flag, p.status, kErrWaitTmemFull)) { ok = false; break; }
      tc_fence_after();
      // pass 1: row max over the tile
      float m_tile = -1.0e30f;
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_S + st * 128 + c * 32 + lane_sel, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float s = __uint_as_float(r[e]);
          if (need_mask) {
            const int key = kv0 + c * 32 + e;
            const bool allowed = key <= qpos && key < p.Tk && (p.window_left < 0 || qpos - key <= p.window_left);
            s = allowed ? s : -1.0e30f;
          }
          m_tile = fmaxf(m_tile, s);
        }
      }
      const float m_new = fmaxf(m_run, m_tile);
      const float alpha = fast_exp2((m_run - m_new) * p.scale_log2);
      const float m_scaled = m_new * p.scale_log2;
      // the P buffer must have been consumed by the PV product two tiles ago
      if (!mbar_wait(&p_empty[st], ph ^ 1, abort_flag, p.status, kErrWaitOther)) { ok = false; break; }
      uint8_t* sP = smem + L::kOffP + st * L::kP;
      float l_tile = 0.0f;
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_S + st * 128 + c * 32 + lane_sel, r);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p0 = fast_exp2(__uint_as_float(r[e]) * p.scale_log2 - m_scaled);
          float p1 = fast_exp2(__uint_as_float(r[e + 1]) * p.scale_log2 - m_scaled);
          if (need_mask) {
            const int key = kv0 + c * 32 + e;
            const bool a0 = key <= qpos && key < p.Tk && (p.window_left < 0 || qpos - key <= p.window_left);
            const bool a1 =
                key + 1 <= qpos && key + 1 < p.Tk && (p.window_left < 0 || qpos - key - 1 <= p.window_left);
            p0 = a0 ? p0 : 0.0f;
            p1 = a1 ? p1 : 0.0f;
          }
          // the row sum uses the rounded probabilities, the same values the PV product sees
          const uint32_t pk = pack_bf16(p0, p1);
          l_tile += bf16_lo(pk) + bf16_hi(pk);
          packed[e / 2] = pk;
        }
        // 32 keys = 4 granules of 16 bytes inside the 64-key chunk (c / 2), starting at granule (c % 2) * 4
        uint8_t* chunk = sP + (c / 2) * (BQ * 128) + row * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int gran = ((c & 1) * 4 + g) ^ (row & 7);
          *reinterpret_cast<uint4*>(chunk + gran * 16) =
              make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
        }
      }
      tc_fence_before();
      fence_async_shared();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[st]);
        mbar_arrive(&p_full[st]);
      }
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
      // fold the previous tile's product into the running output (it was computed relative to the
      // previous maximum, so it is rescaled together with the accumulator)
      if (it > 0) {
        const int pst = (it - 1) & 1;
        const uint32_t pph = ((it - 1) >> 1) & 1;
        if (!mbar_wait(&o_full[pst], pph, abort_flag, p.status, kErrWaitTmemFull)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_O + pst * D + c * 32 + lane_sel, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o_acc[c * 32 + e] = (o_acc[c * 32 + e] * alpha_prev + __uint_as_float(r[e]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_empty[pst]);
      }
      alpha_prev = alpha;
    }
    if (ok) {
      // last tile's product
      const int it = n_tiles - 1;
      const int pst = it & 1;
      const uint32_t pph = (it >> 1) & 1;
      if (mbar_wait(&o_full[pst], pph, abort_flag, p.status, kErrWaitTmemFull)) {
        tc_fence_after();
        const float inv_l = 1.0f / l_run;
        __nv_bfloat16* op = p.O + static_cast<long long>(b) * p.o_stride_b +
                            static_cast<long long>(q0 + row) * p.o_stride_t + static_cast<long long>(h) * p.o_stride_h;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_O + pst * D + c * 32 + lane_sel, r);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = c * 32 + g * 8 + e * 2;
                const float v0 = (o_acc[i] * alpha_prev + __uint_as_float(r[g * 8 + e * 2])) * inv_l;
                const float v1 = (o_acc[i + 1] * alpha_prev + __uint_as_float(r[g * 8 + e * 2 + 1])) * inv_l;
                w[e] = pack_bf16(v0, v1);
              }
              *reinterpret_cast<uint4*>(op + c * 32 + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        if (row_ok) {
          // natural-log statistic: max*scale + log(sum)
          p.lse[(static_cast<long long>(b) * p.H + h) * p.Tq + q0 + row] =
              m_run * p.scale_log2 * 0.6931471805599453f + logf(l_run);
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

}  // namespace

const char* attention_fwd(const AttnArgs& a, cudaStream_t stream) {
  if (a.D != 64 && a.D != 128) return "attention_fwd: head_dim must be 64 or 128";
  if (a.H % a.KVH) return "attention_fwd: heads must be a multiple of kv heads";
  CUtensorMap tq, tk, tv;
  {
    const long long dq[4] = {a.D, a.H, a.Tq, a.B};
    const long long sq[3] = {a.q_stride_h, a.q_stride_t, a.q_stride_b};
    const int box[4] = {64, 1, BQ, 1};
    if (!make_tmap_bf16_4d(&tq, a.Q, dq, sq, box)) return "attention_fwd: tensor map (Q) failed";
    const long long dk[4] = {a.D, a.KVH, a.Tk, a.B};
    const long long sk[3] = {a.k_stride_h, a.k_stride_t, a.k_stride_b};
    const int boxk[4] = {64, 1, BKV, 1};
    if (!make_tmap_bf16_4d(&tk, a.K, dk, sk, boxk)) return "attention_fwd: tensor map (K) failed";
    const long long sv[3] = {a.v_stride_h, a.v_stride_t, a.v_stride_b};
    if (!make_tmap_bf16_4d(&tv, a.V, dk, sv, boxk)) return "attention_fwd: tensor map (V) failed";
  }
  FwdParams p;
  p.B = a.B, p.H = a.H, p.KVH = a.KVH, p.Tq = a.Tq, p.Tk = a.Tk;
  p.q_offset = a.q_offset;
  p.window_left = a.window_left;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.O = static_cast<__nv_bfloat16*>(a.O);
  p.o_stride_b = a.o_stride_b, p.o_stride_t = a.o_stride_t, p.o_stride_h = a.o_stride_h;
  p.lse = a.lse;
  p.status = a.status;
  const dim3 grid((a.Tq + BQ - 1) / BQ, a.H, a.B);
  cudaError_t e;
  if (a.D == 128) {
    static bool cfg = false;
    if (!cfg) {
      e = cudaFuncSetAttribute(attention_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               FwdSmem<128>::kTotal);
      if (e != cudaSuccess) return cudaGetErrorString(e);
      cfg = true;
    }
    attention_fwd_kernel<128><<<grid, NUM_THREADS, FwdSmem<128>::kTotal, stream>>>(tq, tk, tv, p);
  } else {
    static bool cfg = false;
    if (!cfg) {
      e = cudaFuncSetAttribute(attention_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               FwdSmem<64>::kTotal);
      if (e != cudaSuccess) return cudaGetErrorString(e);
      cfg = true;
    }
    attention_fwd_kernel<64><<<grid, NUM_THREADS, FwdSmem<64>::kTotal, stream>>>(tq, tk, tv, p);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nc

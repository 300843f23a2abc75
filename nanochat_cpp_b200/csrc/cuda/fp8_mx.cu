// MXFP8 GEMM for sm_100a: E4M3 operands with one power-of-two scale (UE8M0) per 32 consecutive K elements of every
// row, applied by the tensor core itself (tcgen05.mma kind::mxf8f6f4.block_scale), and its quantizer.
//
// The reference scales fp8 operands per tensor and calls cublasLt (backends/cuda/kernels/fp8.cu:39-80,
// backends/cuda/gemm.cu:553-690). The two-level kernel in fp8.cu applies fp32 block scales on the CUDA cores and
// is bound by that promotion. Here the scales travel with the operands into tensor memory, the whole K extent
// accumulates in TMEM, and the epilogue is the plain bf16 one, so the product runs at the fp8 tensor rate.
//
// Scale layout ("atoms"). The scales of 128 rows x 128 K elements (128 x 4 bytes) form one 512-byte atom in the
// order tcgen05.cp.32x128b.warpx4 expects: byte (r % 32) * 16 + (r / 32) * 4 + k32. Rows are grouped by GEMM tile
// (`tile_rows` = 128 for the activations, the kernel's BN for the weights) so that the atoms of one tile and one
// 128-deep K block are contiguous: atom index = ((r / tile_rows) * (K / 128) + kb) * atoms_per_tile + (r % tile_rows) / 128.
//
//   warp 0       producer: TMA tiles of A (128 x 128 B) and B (BN x 128 B), copies of their scale atoms
//   warp 1       TMEM allocation; per K block: tcgen05.cp of the atoms into TMEM (one K block ahead of their MMAs,
//                four rotating column slots behind the accumulators), 4 MMAs of K = 32 (scale id 0..3)
//   warps 2..9   epilogue: TMEM -> registers -> bf16 -> warp-private shared-memory transpose -> 64-byte row segments
//                (optionally relu(x)^2 as a second output), overlapped with the next tile (two accumulators)
// Two kernels share these roles: one CTA per 128 x BN tile, and (the default for M > 128) CTA pairs computing
// 256 x BN tiles with tcgen05.mma.cta_group::2, where each CTA loads its 128 rows of A, half of the B tile and the
// scale atoms, and the leader issues the copies and the MMAs for both. BN is 192 or 224 (two accumulators plus the
// scale columns must fit the 512 TMEM columns); tiles are visited in groups of row tiles so that operands stay in L2.
#include "fp8.h"

#include <cuda.h>
#include <cuda_fp8.h>

#include "mx_quant.cuh"
#include "ptx.cuh"
#include "tmap.h"

namespace nc {

namespace {

// One half-warp per two consecutive (row, 128-wide K block) units: a thread owns 8 consecutive elements of each,
// four threads share a scale; both 16-byte loads are issued before either unit is processed.
// Rows in [R, R_pad) only get the neutral scale byte 127 (2^0); their data is never read (TMA zero-fills).
// R_pad * (K / 128) is even, so a half-warp's two units are in range together and a warp's shuffles are uniform.
__global__ void __launch_bounds__(256) quantize_mx_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                          uint8_t* __restrict__ xq, uint8_t* __restrict__ sf, int R,
                                                          int R_pad, int K, int tile_rows, int atoms_per_tile) {
  const int kbs = K / 128;
  const uint32_t total = static_cast<uint32_t>(R_pad) * kbs;        // the host checks that this fits 31 bits
  const uint32_t unit0 = (blockIdx.x * 16u + (threadIdx.x >> 4)) * 2u;
  const int l16 = threadIdx.x & 15;
  const int base = threadIdx.x & 16;
  const bool in_range = unit0 < total;
  int row[2], kb[2];
  uint4 raw[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const uint32_t unit = in_range ? unit0 + u : 0u;
    row[u] = static_cast<int>(unit / static_cast<uint32_t>(kbs));
    kb[u] = static_cast<int>(unit - static_cast<uint32_t>(row[u]) * kbs);
    raw[u] = make_uint4(0, 0, 0, 0);
    if (in_range && row[u] < R)
      raw[u] = *reinterpret_cast<const uint4*>(x + static_cast<long long>(row[u]) * ldx + kb[u] * 128 + l16 * 8);
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
    float v[8];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = bf16_lo(w[i]);
      v[2 * i + 1] = bf16_hi(w[i]);
      amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const uint32_t eb = mx_block_exponent(amax);
    const bool live = in_range && row[u] < R;
    if (live) {
      *reinterpret_cast<uint2*>(xq + static_cast<long long>(row[u]) * K + kb[u] * 128 + l16 * 8) =
          mx_pack8(v, mx_inverse_scale(eb));
    }
    // the four scale bytes of this (row, K block) sit in lanes 0, 4, 8, 12 of the half-warp
    const uint32_t b0 = __shfl_sync(0xffffffffu, eb, base), b1 = __shfl_sync(0xffffffffu, eb, base + 4);
    const uint32_t b2 = __shfl_sync(0xffffffffu, eb, base + 8), b3 = __shfl_sync(0xffffffffu, eb, base + 12);
    if (in_range && l16 == 0) {
      const int tile = row[u] / tile_rows, rt = row[u] % tile_rows;
      const long long atom = (static_cast<long long>(tile) * kbs + kb[u]) * atoms_per_tile + rt / 128;
      *reinterpret_cast<uint32_t*>(sf + atom * 512 + mx_atom_offset(rt % 128)) = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
constexpr int BM = 128, BK = 128;             // BK in elements = bytes
constexpr int UMMA_K = 32;
constexpr int A_BYTES = BM * BK;
constexpr int SFA_BYTES = 512, SFB_BYTES = 1024;   // one atom for the 128 A rows, two for the B rows
constexpr int SF_BYTES = SFA_BYTES + SFB_BYTES;
constexpr int EPI_WARPS = 8;
constexpr int NUM_THREADS = 64 + EPI_WARPS * 32;
constexpr int TMEM_COLS = 512;
constexpr int SF_SLOTS = 4, SF_SLOT_COLS = 16;     // scale columns rotate over four slots behind the accumulators
constexpr int kEpiStageBytes = 32 * 64;            // one warp's 32 rows x 32 bf16 on the way out

template <int BN>
struct MxCfg {
  static_assert(BN % 32 == 0 && BN > 128 && 2 * BN + SF_SLOTS * SF_SLOT_COLS <= TMEM_COLS, "tile width");
  static constexpr int B_BYTES = BN * BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;          // a multiple of 1024 (SWIZZLE_128B tiles)
  static constexpr int STAGES = BN <= 192 ? 5 : 4;
  static constexpr int H0 = ((BN / 32 + 1) / 2) * 32;             // columns of the first epilogue half
  static constexpr int SF_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = SF_OFF + STAGES * SF_BYTES;
  static constexpr int EPI_OFF = BAR_OFF + 256;
  static constexpr int SMEM_BYTES = EPI_OFF + EPI_WARPS * kEpiStageBytes + 1024;
  static constexpr int SF_COL0 = 2 * BN;
};

struct MxParams {
  int M, N, K, m_blocks, n_blocks, k_blocks;
  const uint8_t* sfa;
  const uint8_t* sfb;
  __nv_bfloat16* C;
  __nv_bfloat16* C2;
  long long ldc;
  int* status;
  int group_m;
};

// Tile order: groups of `group_m` row tiles sweep all column tiles before the next group starts (rows fastest inside
// a group), so the CTAs running at one time share a few A row tiles and B column tiles that stay in L2, and every
// operand is read from DRAM about once. (With rows fastest over the whole matrix, A is re-read once per column tile.)
__device__ __forceinline__ void mx_decode_unit(const MxParams& p, int unit, int& m_blk, int& n_blk) {
  const int per_group = p.group_m * p.n_blocks;
  const int g = unit / per_group, r = unit - g * per_group;
  const int m_first = g * p.group_m;
  const int gm = min(p.group_m, p.m_blocks - m_first);
  n_blk = r / gm;
  m_blk = m_first + (r - n_blk * gm);
}

// kind::mxf8f6f4 with E4M3 operands (format 0), UE8M0 scales, both operands K-major. The scale ids (which of the
// four bytes of a TMEM scale column this K = 32 step uses) are OR-ed in per instruction.
__host__ __device__ constexpr uint32_t make_idesc_mx_e4m3(int m, int n) {
  return (1u << 23) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ uint32_t with_sf_id(uint32_t idesc, uint32_t id) { return idesc | (id << 29) | (id << 4); }

__device__ __forceinline__ void mma_mxf8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}

// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, replicated into all four lane quadrants.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Ask L2 for a tile some time before a TMA load brings it into shared memory (no shared memory is held meanwhile).
__device__ __forceinline__ void tma_prefetch_l2_2d(const void* tmap, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(tmap)),
               "r"(c0), "r"(c1)
               : "memory");
}

// Unswizzled K-major descriptor of one scale atom: 8-row groups of 16-byte rows, 128 bytes apart.
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const void* tmap, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void mma_mxf8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
// In both CTAs of the pair: 32 rows x 16 bytes of the CTA's own shared memory -> 4 columns of its own TMEM.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// The MMA-issuing thread's loop over this CTA's (or pair's) tiles and K blocks. The scale atoms of K block i + 1
// are copied into tensor memory (their own slot of columns) BEFORE the MMAs of K block i are issued, so the copy's
// latency hides behind those MMAs instead of sitting between two K blocks.
template <bool PAIR, int BN, int STAGES, int STAGE_BYTES, int SF_COL0>
__device__ __forceinline__ void mx_mma_loop(const MxParams& p, int my_units, uint8_t* smem, uint8_t* sf_smem,
                                            uint64_t* full_bar, uint64_t* empty_bar, uint64_t* acc_full,
                                            uint64_t* acc_empty, uint32_t tmem_base, volatile int* abort_flag) {
  constexpr uint32_t idesc = make_idesc_mx_e4m3(PAIR ? 2 * BM : BM, BN);
  const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem), 16, 1024);
  const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(smem) + A_BYTES, 16, 1024);
  const int items = my_units * p.k_blocks;
  auto copy_scales = [&](int st, uint32_t ph, int sl) -> bool {
    if (!mbar_wait(&full_bar[st], ph, abort_flag, p.status, kErrWaitFull)) return false;
    tc_fence_after();
    const uint32_t ss = smem_u32(sf_smem + st * SF_BYTES);
    const uint32_t tsfa = tmem_base + SF_COL0 + sl * SF_SLOT_COLS, tsfb = tsfa + 4;
    if (PAIR) {
      tmem_cp_32x128b_warpx4_pair(tsfa, make_sf_desc(ss));
      tmem_cp_32x128b_warpx4_pair(tsfb, make_sf_desc(ss + SFA_BYTES));
      tmem_cp_32x128b_warpx4_pair(tsfb + 4, make_sf_desc(ss + SFA_BYTES + 512));
    } else {
      tmem_cp_32x128b_warpx4(tsfa, make_sf_desc(ss));
      tmem_cp_32x128b_warpx4(tsfb, make_sf_desc(ss + SFA_BYTES));
      tmem_cp_32x128b_warpx4(tsfb + 4, make_sf_desc(ss + SFA_BYTES + 512));
    }
    return true;
  };
  int stage = 0, slot = 0, buf = 0, kb = 0;
  uint32_t phase = 0, aphase = 0;
  if (items > 0 && !copy_scales(0, 0, 0)) return;
  for (int i = 0; i < items; ++i) {
    int nstage = stage + 1;
    uint32_t nphase = phase;
    if (nstage == STAGES) nstage = 0, nphase ^= 1;
    const int nslot = (slot + 1) & (SF_SLOTS - 1);
    if (kb == 0) {
      if (!mbar_wait(&acc_empty[buf], aphase ^ 1, abort_flag, p.status, kErrWaitTmemEmpty)) return;
      tc_fence_after();
    }
    if (i + 1 < items && !copy_scales(nstage, nphase, nslot)) return;
    const uint32_t tsfa = tmem_base + SF_COL0 + slot * SF_SLOT_COLS, tsfb = tsfa + 4;
    const uint64_t da = a_desc0 + static_cast<uint64_t>(stage * (STAGE_BYTES >> 4));
    const uint64_t db = b_desc0 + static_cast<uint64_t>(stage * (STAGE_BYTES >> 4));
#pragma unroll
    for (int k = 0; k < BK / UMMA_K; ++k) {   // 32 one-byte elements = 32 bytes = 2 descriptor units per step
      if (PAIR)
        mma_mxf8_ss_pair(tmem_base + buf * BN, da + static_cast<uint64_t>(2 * k), db + static_cast<uint64_t>(2 * k),
                         with_sf_id(idesc, k), tsfa, tsfb, (kb | k) ? 1u : 0u);
      else
        mma_mxf8_ss(tmem_base + buf * BN, da + static_cast<uint64_t>(2 * k), db + static_cast<uint64_t>(2 * k),
                    with_sf_id(idesc, k), tsfa, tsfb, (kb | k) ? 1u : 0u);
    }
    if (PAIR) mma_commit_pair(&empty_bar[stage], 3); else mma_commit(&empty_bar[stage]);
    if (++kb == p.k_blocks) {
      kb = 0;
      if (PAIR) mma_commit_pair(&acc_full[buf], 3); else mma_commit(&acc_full[buf]);
      if (++buf == 2) buf = 0, aphase ^= 1;
    }
    stage = nstage, phase = nphase, slot = nslot;
  }
}

// Epilogue of one 128-row accumulator for one warp: the thread owns row `row0 + lane`; the warp covers the columns
// [col_first, col_first + 32 * groups) of the tile that starts at output column n0. A group of 32 columns becomes
// 64 bytes of bf16 per row, goes through a warp-private swizzled tile and leaves as full 64-byte row segments
// (four lanes per row). `release()` runs once, as soon as the whole accumulator is in registers.
template <bool RELU2, int MAX_GROUPS, class Release>
__device__ __forceinline__ void mx_store_tile(const MxParams& p, uint32_t taddr, int row0, int n0, int col_first,
                                              int groups, uint8_t* stage_buf, int lane, Release release) {
  const bool row_ok = row0 + lane < p.M;
  const int rows_valid = min(32, p.M - row0);
  const int g4 = lane & 3;
  auto emit = [&](__nv_bfloat16* base, const uint4 (&v)[4], int c0) {
    if (row_ok) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4*>(stage_buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) = v[j];
    }
    __syncwarp();
    const bool col_ok = c0 + g4 * 8 < p.N;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int rr = it * 8 + (lane >> 2);
      if (col_ok && rr < rows_valid)
        *reinterpret_cast<uint4*>(base + static_cast<long long>(row0 + rr) * p.ldc + c0 + g4 * 8) =
            *reinterpret_cast<const uint4*>(stage_buf + rr * 64 + ((g4 ^ ((rr >> 1) & 3)) << 4));
    }
    __syncwarp();
  };
  uint32_t r[2][32];
  tmem_ld_32x32(taddr + col_first, r[0]);
#pragma unroll
  for (int g = 0; g < MAX_GROUPS; ++g) {
    if (g >= groups) break;
    tmem_ld_wait();
    if (g + 1 < groups) {
      tmem_ld_32x32(taddr + col_first + (g + 1) * 32, r[(g + 1) & 1]);
    } else {
      tc_fence_before();
      __syncwarp();
      release();
    }
    const int c0 = n0 + col_first + g * 32;
    if (c0 >= p.N) continue;
    const uint32_t(&acc)[32] = r[g & 1];
    uint4 outs[4], acts[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t* a8 = acc + j * 8;
      outs[j].x = pack_bf16(__uint_as_float(a8[0]), __uint_as_float(a8[1]));
      outs[j].y = pack_bf16(__uint_as_float(a8[2]), __uint_as_float(a8[3]));
      outs[j].z = pack_bf16(__uint_as_float(a8[4]), __uint_as_float(a8[5]));
      outs[j].w = pack_bf16(__uint_as_float(a8[6]), __uint_as_float(a8[7]));
      if (RELU2) {
        const uint32_t ow[4] = {outs[j].x, outs[j].y, outs[j].z, outs[j].w};
        uint32_t aw[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = fmaxf(bf16_lo(ow[e]), 0.0f), hi = fmaxf(bf16_hi(ow[e]), 0.0f);
          aw[e] = pack_bf16(lo * lo, hi * hi);
        }
        acts[j] = make_uint4(aw[0], aw[1], aw[2], aw[3]);
      }
    }
    if (!RELU2 || p.C != p.C2) emit(p.C, outs, c0);
    if (RELU2) emit(p.C2, acts, c0);
  }
}

template <int BN, bool RELU2>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const MxParams p) {
  using Cfg = MxCfg<BN>;
  constexpr int STAGES = Cfg::STAGES, STAGE_BYTES = Cfg::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sf_smem = smem + Cfg::SF_OFF;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_units = p.m_blocks * p.n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], EPI_WARPS);
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
        int m_blk, n_blk;
      mx_decode_unit(p, unit, m_blk, n_blk);
        const uint8_t* sfa = p.sfa + static_cast<long long>(m_blk) * p.k_blocks * SFA_BYTES;
        const uint8_t* sfb = p.sfb + static_cast<long long>(n_blk) * p.k_blocks * SFB_BYTES;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrWaitEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* ss = sf_smem + stage * SF_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES + SF_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * BK, m_blk * BM);
          tma_load_2d(sa + A_BYTES, &tmB, &full_bar[stage], kb * BK, n_blk * BN);
          bulk_load(ss, sfa + static_cast<long long>(kb) * SFA_BYTES, SFA_BYTES, &full_bar[stage]);
          bulk_load(ss + SFA_BYTES, sfb + static_cast<long long>(kb) * SFB_BYTES, SFB_BYTES, &full_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {   // give the copies in flight time to land before the CTA's shared memory goes away
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const int my_units = blockIdx.x < total_units ? (total_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
      mx_mma_loop<false, BN, STAGES, STAGE_BYTES, Cfg::SF_COL0>(p, my_units, smem, sf_smem, full_bar, empty_bar, acc_full,
                                                                acc_empty, tmem_base, abort_flag);
    }
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    const int col_first = half ? Cfg::H0 : 0;
    const int groups = (half ? BN - Cfg::H0 : Cfg::H0) / 32;
    uint8_t* stage_buf = smem + Cfg::EPI_OFF + (warp - 2) * kEpiStageBytes;
    int buf = 0;
    uint32_t aphase = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
      int m_blk, n_blk;
      mx_decode_unit(p, unit, m_blk, n_blk);
      if (!mbar_wait(&acc_full[buf], aphase, abort_flag, p.status, kErrWaitTmemFull)) break;
      tc_fence_after();
      uint64_t* done = &acc_empty[buf];
      mx_store_tile<RELU2, Cfg::H0 / 32>(p, tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16),
                                         m_blk * BM + q * 32, n_blk * BN, col_first, groups, stage_buf, lane, [&] {
                                           if (lane == 0) mbar_arrive(done);   // the MMA warp may refill this buffer
                                         });
      if (++buf == 2) {
        buf = 0;
        aphase ^= 1;
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
// CTA pairs (cta_group::2): two CTAs of a cluster compute one 256 x BN tile. Each holds its 128 rows of A, its half
// of the B tile (BN / 2 rows), the scale atom of its A rows and the scale atoms of ALL BN columns; the leader issues
// tcgen05.cp and tcgen05.mma for both. Per output element the pair reads (128 + BN / 2) operand rows from L2
// instead of (128 + BN): the single-CTA kernel is bound by L2 bandwidth at the fp8 rate, this one is not.
template <int BN>
struct MxPairCfg {
  static constexpr int B_BYTES = (BN / 2) * BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static_assert(STAGE_BYTES % 1024 == 0, "SWIZZLE_128B tiles start on 1024-byte boundaries");
  static constexpr int STAGES = BN <= 192 ? 7 : 6;                // as many as fit in 227 KB
  static constexpr int H0 = ((BN / 32 + 1) / 2) * 32;
  static constexpr int SF_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = SF_OFF + STAGES * SF_BYTES;
  static constexpr int EPI_OFF = BAR_OFF + 256;
  static constexpr int SMEM_BYTES = EPI_OFF + EPI_WARPS * kEpiStageBytes + 1024;
  static constexpr int SF_COL0 = 2 * BN;
  static_assert(SMEM_BYTES <= 232448, "shared memory per CTA");
};

template <int BN, bool RELU2>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mxfp8_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                       const MxParams p) {   // p.m_blocks counts 256-row tiles
  using Cfg = MxPairCfg<BN>;
  constexpr int STAGES = Cfg::STAGES, STAGE_BYTES = Cfg::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sf_smem = smem + Cfg::SF_OFF;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0 = leader
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int total_units = p.m_blocks * p.n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);    // the leader's arrive.expect_tx; the bytes of both CTAs complete on it
      mbar_init(&empty_bar[s], 1);   // one commit, delivered to both CTAs
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * EPI_WARPS);   // the epilogue warps of both CTAs (used in the leader only)
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmSFA);
    tma_prefetch_desc(&tmSFB);
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
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = pair_id; unit < total_units && ok; unit += num_pairs) {
        int m_blk, n_blk;
      mx_decode_unit(p, unit, m_blk, n_blk);
        const int m0 = m_blk * (2 * BM) + static_cast<int>(rank) * BM;
        const int n0 = n_blk * BN + static_cast<int>(rank) * (BN / 2);
        // rows of 256 bytes in the scale arrays: an atom is two rows
        const int sfa_row0 = (m_blk * 2 + static_cast<int>(rank)) * p.k_blocks * 2;
        const int sfb_row0 = n_blk * p.k_blocks * 4;
        const bool has_next = unit + num_pairs < total_units;
        int m0_next = 0, n0_next = 0;
        if (has_next) {
          int mn, nn;
          mx_decode_unit(p, unit + num_pairs, mn, nn);
          m0_next = mn * (2 * BM) + static_cast<int>(rank) * BM;
          n0_next = nn * BN + static_cast<int>(rank) * (BN / 2);
        }
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrWaitEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* ss = sf_smem + stage * SF_BYTES;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * (STAGE_BYTES + SF_BYTES));
          const uint32_t bar = mapa_u32(&full_bar[stage], 0);
          tma_load_2d_pair(sa, &tmA, bar, kb * BK, m0);
          tma_load_2d_pair(sa + A_BYTES, &tmB, bar, kb * BK, n0);
          tma_load_2d_pair(ss, &tmSFA, bar, 0, sfa_row0 + kb * 2);
          tma_load_2d_pair(ss + SFA_BYTES, &tmSFB, bar, 0, sfb_row0 + kb * 4);
          if (has_next) {   // the same K block of the pair's next tile: in L2 one whole tile ahead of its load
            tma_prefetch_l2_2d(&tmA, kb * BK, m0_next);
            tma_prefetch_l2_2d(&tmB, kb * BK, n0_next);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {   // give the copies in flight time to land before the CTA's shared memory goes away
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const int my_units = pair_id < total_units ? (total_units - pair_id + num_pairs - 1) / num_pairs : 0;
      mx_mma_loop<true, BN, STAGES, STAGE_BYTES, Cfg::SF_COL0>(p, my_units, smem, sf_smem, full_bar, empty_bar, acc_full,
                                                               acc_empty, tmem_base, abort_flag);
    }
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    const int col_first = half ? Cfg::H0 : 0;
    const int groups = (half ? BN - Cfg::H0 : Cfg::H0) / 32;
    uint8_t* stage_buf = smem + Cfg::EPI_OFF + (warp - 2) * kEpiStageBytes;
    const uint32_t leader_empty[2] = {mapa_u32(&acc_empty[0], 0), mapa_u32(&acc_empty[1], 0)};
    int buf = 0;
    uint32_t aphase = 0;
    for (int unit = pair_id; unit < total_units; unit += num_pairs) {
      int m_blk, n_blk;
      mx_decode_unit(p, unit, m_blk, n_blk);
      if (!mbar_wait(&acc_full[buf], aphase, abort_flag, p.status, kErrWaitTmemFull)) break;
      tc_fence_after();
      const uint32_t done = leader_empty[buf];
      mx_store_tile<RELU2, Cfg::H0 / 32>(p, tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16),
                                         m_blk * (2 * BM) + static_cast<int>(rank) * BM + q * 32, n_blk * BN, col_first,
                                         groups, stage_buf, lane, [&] {
                                           if (lane == 0) mbar_arrive_cluster(done);
                                         });
      if (++buf == 2) {
        buf = 0;
        aphase ^= 1;
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

template <int BN, bool RELU2>
cudaError_t launch_mx_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb,
                           const MxParams& p, int pairs, cudaStream_t stream) {
  auto kernel = gemm_mxfp8_pair_kernel<BN, RELU2>;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MxPairCfg<BN>::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = MxPairCfg<BN>::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, ta, tb, tsa, tsb, p);
}

template <int BN, bool RELU2>
cudaError_t launch_mx(const CUtensorMap& ta, const CUtensorMap& tb, const MxParams& p, int grid, cudaStream_t stream) {
  // set on every launch: the attribute belongs to the current device's copy of the function
  const cudaError_t e = cudaFuncSetAttribute(gemm_mxfp8_kernel<BN, RELU2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             MxCfg<BN>::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  gemm_mxfp8_kernel<BN, RELU2><<<grid, NUM_THREADS, MxCfg<BN>::SMEM_BYTES, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

}  // namespace

int mxfp8_tile_n(int N) {
  const int pad192 = (N + 191) / 192 * 192, pad224 = (N + 223) / 224 * 224;
  return pad192 < pad224 ? 192 : 224;
}

long long mxfp8_scale_bytes(int R, int K, int tile_rows) {
  const long long tiles = (R + tile_rows - 1) / tile_rows, atoms = (tile_rows + 127) / 128;
  return tiles * atoms * (K / 128) * 512;
}

const char* quantize_mxfp8(const __nv_bfloat16* x, long long ldx, uint8_t* xq, uint8_t* sf, int R, int K, int tile_rows,
                           cudaStream_t s) {
  if (R <= 0 || K <= 0) return nullptr;
  if (K % 128 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return "quantize_mxfp8: K % 128, ld % 8 and 16-byte rows";
  if (tile_rows != 128 && tile_rows != 192 && tile_rows != 224) return "quantize_mxfp8: tile_rows must be 128, 192 or 224";
  const int tiles = (R + tile_rows - 1) / tile_rows, atoms = (tile_rows + 127) / 128;
  const int R_pad = tiles * tile_rows;
  const long long units = static_cast<long long>(R_pad) * (K / 128);
  if (units >= (1ll << 31)) return "quantize_mxfp8: more than 2^31 row blocks";
  quantize_mx_kernel<<<static_cast<unsigned>((units + 31) / 32), 256, 0, s>>>(x, ldx, xq, sf, R, R_pad, K, tile_rows, atoms);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* gemm_mxfp8(const MxGemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return nullptr;
  if (a.K % 128) return "gemm_mxfp8: K must be a multiple of 128";
  if (a.N % 8 || a.ldc % 8) return "gemm_mxfp8: N and ldc must allow 16-byte stores";
  if ((reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.B) | reinterpret_cast<uintptr_t>(a.sfa) |
       reinterpret_cast<uintptr_t>(a.sfb) | reinterpret_cast<uintptr_t>(a.C) | reinterpret_cast<uintptr_t>(a.C2)) & 15)
    return "gemm_mxfp8: misaligned operand";
  const int bn = mxfp8_tile_n(a.N);
  const bool pair = a.variant == 2 || (a.variant == 0 && a.M > BM);
  MxParams p;
  p.M = a.M, p.N = a.N, p.K = a.K;
  p.n_blocks = (a.N + bn - 1) / bn, p.k_blocks = a.K / BK;
  p.sfa = a.sfa, p.sfb = a.sfb;
  p.C = a.C, p.C2 = a.C2, p.ldc = a.ldc, p.status = a.status;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  CUtensorMap ta, tb;
  cudaError_t e;
  if (pair) {
    CUtensorMap tsa, tsb;
    const long long rows_a = mxfp8_scale_bytes(a.M, a.K, BM) / 256, rows_b = mxfp8_scale_bytes(a.N, a.K, bn) / 256;
    if (!make_tmap_u8_2d(&ta, a.A, a.K, a.M, a.K, BK, BM) || !make_tmap_u8_2d(&tb, a.B, a.K, a.N, a.K, BK, bn / 2) ||
        !make_tmap_u8_2d_plain(&tsa, a.sfa, 256, rows_a, 256, 256, 2) ||
        !make_tmap_u8_2d_plain(&tsb, a.sfb, 256, rows_b, 256, 256, 4))
      return "gemm_mxfp8: cuTensorMapEncodeTiled failed";
    p.m_blocks = (a.M + 2 * BM - 1) / (2 * BM);
    p.group_m = 8;
    const int units = p.m_blocks * p.n_blocks;
    const int pairs = units < sms / 2 ? units : sms / 2;
    if (bn == 192)
      e = a.C2 ? launch_mx_pair<192, true>(ta, tb, tsa, tsb, p, pairs, stream)
               : launch_mx_pair<192, false>(ta, tb, tsa, tsb, p, pairs, stream);
    else
      e = a.C2 ? launch_mx_pair<224, true>(ta, tb, tsa, tsb, p, pairs, stream)
               : launch_mx_pair<224, false>(ta, tb, tsa, tsb, p, pairs, stream);
  } else {
    if (!make_tmap_u8_2d(&ta, a.A, a.K, a.M, a.K, BK, BM) || !make_tmap_u8_2d(&tb, a.B, a.K, a.N, a.K, BK, bn))
      return "gemm_mxfp8: cuTensorMapEncodeTiled failed";
    p.m_blocks = (a.M + BM - 1) / BM;
    p.group_m = 16;
    const int units = p.m_blocks * p.n_blocks;
    const int grid = units < sms ? units : sms;
    if (bn == 192)
      e = a.C2 ? launch_mx<192, true>(ta, tb, p, grid, stream) : launch_mx<192, false>(ta, tb, p, grid, stream);
    else
      e = a.C2 ? launch_mx<224, true>(ta, tb, p, grid, stream) : launch_mx<224, false>(ta, tb, p, grid, stream);
  }
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace nc

// Host interface of the block-scaled fp8 path (fp8.cu): E4M3 operands, fp32 scales, bf16 output.
//   activations  x[M,K]  -> xq[M,K] e4m3 + sx[K/128][M]       one scale per row and 128-wide K block
//   weights      w[N,K]  -> wq[N,K] e4m3 + sw[N/128][K/128]   one scale per 128 x 128 block
//   C[M,N] = bf16( sum_kb sx[kb][m] * sw[n/128][kb] * (xq[m, kb-block] . wq[n, kb-block]) )
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nc {

// K must be a multiple of 128. Scales are amax / 448 (1 when the block is all zero).
void quantize_rows_1x128(const __nv_bfloat16* x, long long ldx, uint8_t* xq, float* scales_kb_major, int M, int K,
                         cudaStream_t s);
// N and K multiples of 128.
void quantize_blocks_128x128(const __nv_bfloat16* w, long long ldw, uint8_t* wq, float* scales, int N, int K,
                             cudaStream_t s);

struct Fp8GemmArgs {
  const uint8_t* A = nullptr;   // [M, K] e4m3, row-major
  const uint8_t* B = nullptr;   // [N, K] e4m3, row-major
  const float* scale_a = nullptr;  // [K/128][M]
  const float* scale_b = nullptr;  // [ceil(N/128)][K/128]
  int M = 0, N = 0, K = 0;
  __nv_bfloat16* C = nullptr;   // [M, N]
  long long ldc = 0;
  __nv_bfloat16* C2 = nullptr;  // optional second output relu(C)^2 (same layout)
  int* status = nullptr;
};
// Returns nullptr on success or a static error string.
const char* gemm_fp8_blockscaled(const Fp8GemmArgs& args, cudaStream_t stream);

// ---- MXFP8 (fp8_mx.cu): E4M3 operands, one UE8M0 (power-of-two) scale per row and 32 K elements, applied by
// tcgen05.mma kind::mxf8f6f4.block_scale; the whole K extent accumulates in tensor memory.
// Scales are stored as 512-byte atoms (128 rows x 4 scales, byte (r % 32) * 16 + (r / 32) * 4 + k32), rows grouped
// by GEMM tile: atom = ((r / tile_rows) * (K / 128) + kb) * ceil(tile_rows / 128) + (r % tile_rows) / 128.
// tile_rows is 128 for the A operand and mxfp8_tile_n(N) for the B operand.
int mxfp8_tile_n(int N);
long long mxfp8_scale_bytes(int R, int K, int tile_rows);
// K % 128 == 0, ldx % 8 == 0. Returns nullptr on success or a static error string.
const char* quantize_mxfp8(const __nv_bfloat16* x, long long ldx, uint8_t* xq, uint8_t* sf, int R, int K, int tile_rows,
                           cudaStream_t s);

struct MxGemmArgs {
  const uint8_t* A = nullptr;    // [M, K] e4m3, row-major
  const uint8_t* B = nullptr;    // [N, K] e4m3, row-major
  const uint8_t* sfa = nullptr;  // atoms of A, tile_rows = 128
  const uint8_t* sfb = nullptr;  // atoms of B, tile_rows = mxfp8_tile_n(N)
  int M = 0, N = 0, K = 0;
  __nv_bfloat16* C = nullptr;    // [M, N]
  long long ldc = 0;
  __nv_bfloat16* C2 = nullptr;   // optional second output relu(C)^2 (same layout); C2 == C keeps only the activation
  int* status = nullptr;
  int variant = 0;               // 0: CTA pairs (256-row tiles) when M > 128; 1: single CTAs; 2: CTA pairs
};
const char* gemm_mxfp8(const MxGemmArgs& args, cudaStream_t stream);

}  // namespace nc

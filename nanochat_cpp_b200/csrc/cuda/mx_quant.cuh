// Device helpers shared by the MXFP8 quantizer (fp8_mx.cu) and the row kernels that emit MXFP8 beside their bf16
// output (rowops.cu): the UE8M0 exponent of a 32-element block and the E4M3 packing of eight scaled values.
#pragma once
#include <cuda_fp8.h>
#include <stdint.h>

namespace nc {

// Biased exponent b of the smallest power of two 2^(b - 127) >= amax / 448 (127 for an all-zero block).
__device__ __forceinline__ uint32_t mx_block_exponent(float amax) {
  const uint32_t bits = __float_as_uint(amax * (1.0f / 448.0f));
  const uint32_t eb = (bits >> 23) + ((bits & 0x7fffffu) ? 1u : 0u);
  return amax > 0.0f ? min(max(eb, 1u), 253u) : 127u;
}
// 1 / 2^(b - 127)
__device__ __forceinline__ float mx_inverse_scale(uint32_t eb) { return __uint_as_float((254u - eb) << 23); }

// two values -> two E4M3 bytes (a in bits 0..7, b in bits 8..15), round to nearest even, saturating
__device__ __forceinline__ uint32_t mx_to_e4m3x2(float a, float b) {
  return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ uint2 mx_pack8(const float (&v)[8], float inv) {
  return make_uint2(mx_to_e4m3x2(v[0] * inv, v[1] * inv) | (mx_to_e4m3x2(v[2] * inv, v[3] * inv) << 16),
                    mx_to_e4m3x2(v[4] * inv, v[5] * inv) | (mx_to_e4m3x2(v[6] * inv, v[7] * inv) << 16));
}
// Byte offset of the four scales of (row r of a 128-row group, one 128-deep K block) inside their 512-byte atom.
__device__ __forceinline__ int mx_atom_offset(int r128) { return (r128 & 31) * 16 + (r128 >> 5) * 4; }

}  // namespace nc

// Cached construction of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's driver entry
// point, so the extension does not link libcuda). All maps use the 128-byte swizzle and zero OOB fill.
#pragma once
#include <cuda.h>

namespace nc {

// 3-D bf16 map {d0 (contiguous), d1, d2}; strides s1, s2 in elements; box {box0, box1, 1}.
bool make_tmap_bf16_3d(CUtensorMap* out, const void* ptr, long long d0, long long d1, long long d2, long long s1,
                       long long s2, int box0, int box1);
// 4-D bf16 map; dims[0] is contiguous; strides[i] (elements) belongs to dims[i + 1].
bool make_tmap_bf16_4d(CUtensorMap* out, const void* ptr, const long long dims[4], const long long strides[3],
                       const int box[4]);
// 2-D map of 1-byte elements (fp8 operands): {d0 contiguous, d1}, row stride s1 bytes.
bool make_tmap_u8_2d(CUtensorMap* out, const void* ptr, long long d0, long long d1, long long s1, int box0, int box1);
// the same without shared-memory swizzling: box rows land back to back (box0 <= 256 bytes)
bool make_tmap_u8_2d_plain(CUtensorMap* out, const void* ptr, long long d0, long long d1, long long s1, int box0,
                           int box1);

}  // namespace nc

#include "tmap.h"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace nc {

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(sym);
    }
  });
  return fn;
}

struct Key {
  long long v[14];
  bool operator==(const Key& o) const { return std::memcmp(v, o.v, sizeof(v)) == 0; }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    size_t h = 1469598103934665603ull;
    for (long long x : k.v) {
      h ^= static_cast<size_t>(x);
      h *= 1099511628211ull;
    }
    return h;
  }
};

bool encode_cached(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, int rank, const void* ptr,
                   const long long* dims, const long long* strides, const int* box,
                   CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  static std::mutex mu;
  static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
  Key key;
  std::memset(&key, 0, sizeof(key));
  key.v[0] = reinterpret_cast<long long>(ptr);
  key.v[1] = static_cast<long long>(dt) * 16 + rank + static_cast<long long>(swizzle) * 4096;
  for (int i = 0; i < rank; ++i) {
    key.v[2 + i] = dims[i];
    key.v[10 + i] = box[i];
  }
  for (int i = 0; i < rank - 1; ++i) key.v[6 + i] = strides[i];
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  EncodeFn encode = get_encode();
  if (encode == nullptr) return false;
  cuuint64_t d[5];
  cuuint64_t s[4];
  cuuint32_t b[5], e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = static_cast<cuuint64_t>(dims[i]);
    b[i] = static_cast<cuuint32_t>(box[i]);
    e[i] = 1;
  }
  for (int i = 0; i < rank - 1; ++i) s[i] = static_cast<cuuint64_t>(strides[i]) * elem_bytes;
  const CUresult r = encode(out, dt, rank, const_cast<void*>(ptr), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return true;
}

}  // namespace

bool make_tmap_bf16_3d(CUtensorMap* out, const void* ptr, long long d0, long long d1, long long d2, long long s1,
                       long long s2, int box0, int box1) {
  const long long dims[3] = {d0, d1, d2};
  const long long strides[2] = {s1, s2};
  const int box[3] = {box0, box1, 1};
  return encode_cached(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 3, ptr, dims, strides, box);
}

bool make_tmap_bf16_4d(CUtensorMap* out, const void* ptr, const long long dims[4], const long long strides[3],
                       const int box[4]) {
  return encode_cached(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 4, ptr, dims, strides, box);
}

bool make_tmap_u8_2d(CUtensorMap* out, const void* ptr, long long d0, long long d1, long long s1, int box0, int box1) {
  const long long dims[2] = {d0, d1};
  const long long strides[1] = {s1};
  const int box[2] = {box0, box1};
  return encode_cached(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 2, ptr, dims, strides, box);
}


bool make_tmap_u8_2d_plain(CUtensorMap* out, const void* ptr, long long d0, long long d1, long long s1, int box0,
                           int box1) {
  const long long dims[2] = {d0, d1};
  const long long strides[1] = {s1};
  const int box[2] = {box0, box1};
  return encode_cached(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

}  // namespace nc

// Paged decode attention through a C symbol, with its scratch in a fixed device array (see decode_noalloc.h for
// who needs this and for the rules of use). The kernels are the ones of decode.cu, reached through
// nc::paged_decode_attention, which only launches.
#include "decode_noalloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <climits>
#include <cstdint>
#include <cstdio>
#include <mutex>

#include "decode.h"

namespace {

// Partial sums of the key splits: first B*H*splits*D floats of accumulators, then B*H*splits*2 floats of
// (running maximum, running sum). In host code this name is only a handle for cudaGetSymbolAddress.
static __device__ __align__(256) float g_decode_scratch[NC_DECODE_NOALLOC_MAX_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mutex;

void say(char* message, int len, const char* text) {
  if (message != nullptr && len > 0) std::snprintf(message, static_cast<size_t>(len), "%s", text);
}

// Device address of the array on the current device; looked up on the first call per device.
cudaError_t scratch_for_current_device(float** ptr) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_decode_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_ptr[dev] = p;
  }
  *ptr = g_scratch_ptr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" int nc_paged_decode_attention_splits(int B, int KV, int max_pages, int page_size, int window_left) {
  if (B <= 0 || KV <= 0 || max_pages <= 0 || page_size <= 0) return 1;
  long long keys = static_cast<long long>(max_pages) * page_size;
  if (keys > INT_MAX) keys = INT_MAX;
  if (window_left >= 0 && window_left + 1 < keys) keys = window_left + 1;
  return nc::decode_splits(B, KV, static_cast<int>(keys));
}

extern "C" int nc_paged_decode_attention_noalloc(const void* q, const void* k_pool, const void* v_pool,
                                                 const int* page_table, const int* seq_lens, void* out, int B,
                                                 int H, int KV, int D, int max_pages, int page_size,
                                                 int window_left, float scale, int splits, void* stream,
                                                 char* message, int message_len) {
  if (q == nullptr || k_pool == nullptr || v_pool == nullptr || page_table == nullptr || seq_lens == nullptr ||
      out == nullptr) {
    say(message, message_len, "a required pointer is null");
    return NC_DECODE_NOALLOC_BAD_ARGUMENT;
  }
  if (B <= 0 || H <= 0 || KV <= 0 || max_pages <= 0 || page_size <= 0 || H % KV != 0 || (D != 64 && D != 128)) {
    say(message, message_len, "sizes must be positive, H a multiple of KV and D 64 or 128");
    return NC_DECODE_NOALLOC_BAD_ARGUMENT;
  }
  const int group = H / KV;
  if (group != 1 && group != 2 && group != 4 && group != 8) {
    say(message, message_len, "the group size H / KV must be 1, 2, 4 or 8");
    return NC_DECODE_NOALLOC_BAD_ARGUMENT;
  }
  if (static_cast<long long>(max_pages) * page_size > INT_MAX) {
    say(message, message_len, "max_pages * page_size does not fit a 32-bit key index");
    return NC_DECODE_NOALLOC_BAD_ARGUMENT;
  }
  // the kernels read q, K and V rows with 16-byte loads and write the output with 16-byte-aligned rows
  if (((reinterpret_cast<std::uintptr_t>(q) | reinterpret_cast<std::uintptr_t>(k_pool) |
        reinterpret_cast<std::uintptr_t>(v_pool) | reinterpret_cast<std::uintptr_t>(out)) & 15u) != 0 ||
      ((reinterpret_cast<std::uintptr_t>(page_table) | reinterpret_cast<std::uintptr_t>(seq_lens)) & 3u) != 0) {
    say(message, message_len, "q, k_pool, v_pool and out must be 16-byte aligned; page_table and seq_lens 4-byte aligned");
    return NC_DECODE_NOALLOC_BAD_ARGUMENT;
  }
  if (splits <= 0) splits = nc_paged_decode_attention_splits(B, KV, max_pages, page_size, window_left);
  const long long need = splits > 1 ? static_cast<long long>(B) * H * splits * (D + 2) : 0;
  if (need > NC_DECODE_NOALLOC_MAX_FLOATS) {
    char buf[160];
    std::snprintf(buf, sizeof(buf), "needs %lld scratch floats (B*H*splits*(D+2)); the fixed array holds %d", need,
                  NC_DECODE_NOALLOC_MAX_FLOATS);
    say(message, message_len, buf);
    return NC_DECODE_NOALLOC_TOO_LARGE;
  }
  float* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) {
    say(message, message_len, cudaGetErrorString(e));
    return NC_DECODE_NOALLOC_CUDA_ERROR;
  }
  nc::DecodeArgs a;
  a.B = B, a.H = H, a.KV = KV, a.D = D;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.k_pool = static_cast<const __nv_bfloat16*>(k_pool);
  a.v_pool = static_cast<const __nv_bfloat16*>(v_pool);
  a.page_table = page_table;
  a.max_pages = max_pages;
  a.page_size = page_size;
  a.seq_lens = seq_lens;
  a.window_left = window_left;
  a.scale = scale;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.splits = splits;
  if (splits > 1) {
    a.part_acc = scratch;
    a.part_ml = scratch + static_cast<long long>(B) * H * splits * D;
  }
  const char* err = nc::paged_decode_attention(a, static_cast<cudaStream_t>(stream));
  if (err != nullptr) {
    say(message, message_len, err);
    return NC_DECODE_NOALLOC_CUDA_ERROR;
  }
  return NC_DECODE_NOALLOC_OK;
}

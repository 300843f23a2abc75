// Host-side execution of CUDA-core kernels: the real `.cu` source of the row / optimizer / decode kernels is compiled
// by the host compiler with this header in front of it, and a launch runs every CUDA thread of a block as a fiber
// on the calling OS thread. A machine without a GPU can then run the kernels' own code against the CPU definitions
// of the operators (tests/test_kernel_emu_cpu.py) - index arithmetic, tails, masks, reductions and the order of
// barriers are what the device executes, only the instruction set differs.
//
// What is emulated: the thread hierarchy (gridDim / blockIdx / blockDim / threadIdx), static and dynamic shared
// memory, __syncthreads / __syncwarp, warp shuffles and votes (lanes of a warp rendezvous, then exchange), atomics
// (blocks run one after another, so they are plain read-modify-writes), the bf16 / fp8 conversions of the CUDA
// headers' host paths, and the handful of math intrinsics the kernels use. Inline PTX in a kernel needs a
// `#ifdef NC_EMU` alternative beside it. What is not: tcgen05, TMEM, TMA and mbarriers - the tensor-core kernels
// have no host form and are tested on the device only.
//
// The reference has an emulator of the same kind for its own kernels (tools/cuda_sim/emu/cuda_emu.h: fibers per CUDA
// thread, wmma / cp.async / wgmma mapped to host code).
#pragma once
#ifndef NC_EMU
#error "cuda_emu.h is for host builds of kernel sources (define NC_EMU)"
#endif

// the CUDA headers keep a qualifier that is already defined: these win
#define __global__
#define __device__
#define __host__
#define __shared__ static thread_local
#define __constant__ static
#define __grid_constant__
#define __launch_bounds__(...)

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>      // before the macros below: its own declarations use these names as parameters
#include <vector_functions.h>
#include <vector_types.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>

namespace emu {

struct Dim {
  unsigned x = 1, y = 1, z = 1;
};
// The running fiber's coordinates (set by the scheduler every time it resumes a fiber).
struct ThreadState {
  Dim grid, block_idx, block_dim, thread_idx;
};
ThreadState& self();

void sync_block();                          // __syncthreads
void sync_warp(unsigned mask);              // __syncwarp, and the rendezvous inside shuffles / votes
uint32_t exchange(uint32_t mine, int src_lane, unsigned mask);   // value of lane `src_lane` of the caller's warp
unsigned vote(bool pred, unsigned mask);    // ballot
void* dynamic_shared();                     // base of the block's dynamic shared memory

// Runs `body` once per CUDA thread of a grid (blocks one after another, threads of a block as fibers).
void launch(Dim grid, Dim block, size_t dynamic_shared_bytes, const std::function<void()>& body);

}  // namespace emu

#define gridDim (emu::self().grid)
#define blockIdx (emu::self().block_idx)
#define blockDim (emu::self().block_dim)
#define threadIdx (emu::self().thread_idx)
#define warpSize 32

inline void __syncthreads() { emu::sync_block(); }
inline void __syncwarp(unsigned mask = 0xffffffffu) { emu::sync_warp(mask); }

template <typename T>
inline T emu_shfl(T v, int src, unsigned mask) {
  static_assert(sizeof(T) == 4 || sizeof(T) == 8, "shuffle of 4- or 8-byte values");
  if constexpr (sizeof(T) == 4) {
    uint32_t bits;
    std::memcpy(&bits, &v, 4);
    bits = emu::exchange(bits, src, mask);
    std::memcpy(&v, &bits, 4);
  } else {
    uint32_t w[2];
    std::memcpy(w, &v, 8);
    w[0] = emu::exchange(w[0], src, mask);
    w[1] = emu::exchange(w[1], src, mask);
    std::memcpy(&v, w, 8);
  }
  return v;
}
inline int emu_lane() {
  const emu::ThreadState& t = emu::self();
  return static_cast<int>((t.thread_idx.x + t.block_dim.x * (t.thread_idx.y + t.block_dim.y * t.thread_idx.z)) & 31u);
}
template <typename T>
inline T __shfl_xor_sync(unsigned mask, T v, int lane_mask, int width = 32) {
  (void)width;
  return emu_shfl(v, emu_lane() ^ lane_mask, mask);
}
template <typename T>
inline T __shfl_sync(unsigned mask, T v, int src, int width = 32) {
  const int lane = emu_lane();
  return emu_shfl(v, (lane & ~(width - 1)) | (src & (width - 1)), mask);
}
template <typename T>
inline T __shfl_down_sync(unsigned mask, T v, unsigned delta, int width = 32) {
  const int lane = emu_lane();
  const int src = lane + static_cast<int>(delta);
  return emu_shfl(v, (src & (width - 1)) >= (lane & (width - 1)) && src < 32 ? src : lane, mask);
}
inline unsigned __ballot_sync(unsigned mask, int pred) { return emu::vote(pred != 0, mask); }
inline int __any_sync(unsigned mask, int pred) { return emu::vote(pred != 0, mask) != 0; }
inline int __all_sync(unsigned mask, int pred) { return emu::vote(pred != 0, mask) == (mask); }

// atomics: one block at a time, fibers switch only at barriers
template <typename T>
inline T atomicAdd(T* p, T v) {
  const T old = *p;
  *p = old + v;
  return old;
}
inline int atomicCAS(int* p, int expected, int desired) {
  const int old = *p;
  if (old == expected) *p = desired;
  return old;
}
inline float atomicMax(int* p, int v) {
  const int old = *p;
  *p = std::max(old, v);
  return old;
}

// math and bit casts (device spellings)
inline float __expf(float x) { return std::exp(x); }
inline float __logf(float x) { return std::log(x); }
inline float __fdividef(float a, float b) { return a / b; }
inline float rsqrtf(float x) { return 1.0f / std::sqrt(x); }
inline float __frcp_rn(float x) { return 1.0f / x; }
inline float __uint_as_float(uint32_t u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint32_t __float_as_uint(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}
inline int __float_as_int(float f) { return static_cast<int>(__float_as_uint(f)); }
inline float __int_as_float(int i) { return __uint_as_float(static_cast<uint32_t>(i)); }
template <typename T>
inline T __ldg(const T* p) { return *p; }
template <typename T>
inline T __ldcs(const T* p) { return *p; }
template <typename T>
inline void __stcs(T* p, T v) { *p = v; }
using std::max;
using std::min;

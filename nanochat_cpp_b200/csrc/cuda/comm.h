// Host launchers of the data-parallel communication kernels (comm.cu). All of them work on symmetric
// buffers: every rank allocated the same layout, `PeerPtrs` holds the address of that buffer on each
// rank (peer addresses are NVLink peer mappings; entry [rank] is the local buffer).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace nc {

constexpr int kMaxRanks = 8;

struct PeerPtrs {
  void* p[kMaxRanks];
  void* mc = nullptr;   // NVLink multicast address of the same (symmetric) buffer, or null: see store_all16 in comm.cu
};

struct Segment {
  long long offset;  // elements from the start of the flat buffer
  long long count;   // elements (multiple of 4)
};

// Publish `value` into slot `slot` of every rank's flag array: flags[slot * world + my_rank] = value.
void comm_signal(const PeerPtrs& flags, int world, int my_rank, int slot, int value, cudaStream_t s);

// Spin (bounded) until flags[slot * world + r] >= value for every r; records kErrWaitPeer on expiry.
// `budget_ms` <= 0: the default peer-wait budget (20 s). On expiry the status word becomes kErrWaitPeer and the
// kernel returns; the context stays usable.
void comm_wait(const int* local_flags, int world, int slot, int value, int* status, cudaStream_t s,
               int budget_ms = 0);

// Gradient reduce-scatter by peer loads: for every element of this rank's segments,
//   out[e] = scale * sum_{r = 0..world-1} grads[r][e]   (fixed rank order)
// written in place into the local gradient buffer, plus the sum of squares of the result accumulated
// into `sumsq` (double). Waits first until every rank has published `value` in `slot`.
void comm_reduce_pull(const PeerPtrs& grads, int world, int my_rank, const Segment* segs_dev, int nsegs,
                      long long total, float scale, const int* local_flags, int slot, int value, double* sumsq,
                      int* status, int ctas, cudaStream_t s);

// Reduce-scatter with bf16 on the wire, first half: the elements of this rank's gradient that other ranks own are
// scaled, rounded to bf16 and stored into the owners' receive buffers (`recv.p[owner] + my_rank * recv_stride +
// position`). `segs_dev`: int64 [nsegs, 5] rows (first vector index, source element offset, destination position,
// destination rank, element count); a vector is 8 elements, `nvec` vectors in all. At most 128 rows per launch.
void comm_grad_push(const float* grad, const PeerPtrs& recv, long long recv_stride, int my_rank,
                    const long long* segs_dev, int nsegs, long long nvec, float scale, int ctas, cudaStream_t s);

// Second half, on the owner: waits (bounded) for `value` in `slot` from every rank, then for every owned element
//   grad[e] = scale * grad[e] + sum_{r != my_rank} recv[r * recv_stride + position]     (fixed rank order, fp32)
// and accumulates the sum of squares of the result into `sumsq`. `segs_dev`: int64 [nsegs, 4] rows (first vector
// index, gradient element offset, receive position, element count). At most 64 rows per launch.
void comm_grad_reduce_local(float* grad, const __nv_bfloat16* recv, long long recv_stride, int world, int my_rank,
                            const long long* segs_dev, int nsegs, long long nvec, float scale,
                            const int* local_flags, int slot, int value, double* sumsq, int* status, int ctas,
                            cudaStream_t s);

// AdamW on this rank's slice, writing the updated bf16 values into every rank's parameter buffer
// (values.p[r] + value_offset): the all-gather is the update's store.
void comm_adamw_push(float* master, const PeerPtrs& values, long long value_offset, int world, const float* grad,
                     float* m, float* v, long long n, float lr, float beta1, float beta2, float eps,
                     float weight_decay, int step, const float* grad_scale, cudaStream_t s, int max_ctas = 0);

// Muon's last stage (cautious decay + update) for one matrix, pushing the bf16 result to every rank.
void comm_muon_apply_push(float* master, const PeerPtrs& values, long long value_offset, int world,
                          const __nv_bfloat16* xb, const float* scale0, const float* line_scale,
                          bool lines_are_rows, int rows, int cols, float lr, float weight_decay, cudaStream_t s);

// The same for a whole shape group in one launch (cols % 8 == 0, every value offset a multiple of 8): `master_ptrs`
// and `value_offsets` are device arrays of P entries.
void comm_muon_apply_push_batched(const long long* master_ptrs, const long long* value_offsets, const PeerPtrs& values,
                                  int world, const __nv_bfloat16* xb, const float* scale0, const float* line_scale,
                                  bool lines_are_rows, int P, int rows, int cols, float lr, float weight_decay,
                                  cudaStream_t s);

}  // namespace nc

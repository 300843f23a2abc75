// Host entry points for the data-parallel transport kernels (csrc/cuda/comm.cu compiled over cuda_emu.h). "Ranks" are
// buffers of one process: a test runs every rank's push, then every owner's reduction, the way the streams of real
// ranks order them, and can leave a flag unset to see a bounded wait give up.
#define NC_EMU
#include "../cuda/comm.cu"

namespace {
nc::PeerPtrs Peers(const long long* ptrs, int n) {
  nc::PeerPtrs p;
  for (int i = 0; i < nc::kMaxRanks; ++i) p.p[i] = nullptr;
  for (int i = 0; i < n && i < nc::kMaxRanks; ++i) p.p[i] = reinterpret_cast<void*>(static_cast<uintptr_t>(ptrs[i]));
  p.mc = nullptr;
  return p;
}
emu::Dim D1(long long n) { return emu::Dim{static_cast<unsigned>(n), 1, 1}; }
}  // namespace

extern "C" {

void nc_emu_comm_signal(const long long* flag_ptrs, int world, int my_rank, int slot, int value) {
  const nc::PeerPtrs flags = Peers(flag_ptrs, world);
  emu::launch(D1(1), D1(32), 0, [&] { nc::signal_kernel(flags, world, my_rank, slot, value); });
}

// Returns after the wait: *status is 0, or 5 when the budget ran out first.
void nc_emu_comm_wait(const int* flags, int world, int slot, int value, int* status, unsigned long long budget_ns) {
  emu::launch(D1(1), D1(32), 0, [&] { nc::wait_kernel(flags, world, slot, value, status, budget_ns); });
}

// segs: rows of five int64 (first_vec, src_off, dst_pos, dst_rank, count), as the transport builds them.
void nc_emu_grad_push(const float* grad, const long long* recv_ptrs, int world, long long recv_stride, int my_rank,
                      const long long* segs, int nsegs, long long nvec, float scale, int ctas) {
  const nc::PeerPtrs recv = Peers(recv_ptrs, world);
  emu::launch(D1(ctas), D1(256), 0, [&] {
    nc::grad_push_kernel(grad, recv, recv_stride, my_rank, reinterpret_cast<const nc::PushSeg*>(segs), nsegs, nvec, scale);
  });
}

// segs: rows of four int64 (first_vec, off, pos, count).
void nc_emu_grad_reduce_local(float* grad, const void* recv, long long recv_stride, int world, int my_rank,
                              const long long* segs, int nsegs, long long nvec, float scale, const int* flags, int slot,
                              int value, double* sumsq, int* status, int ctas) {
  emu::launch(D1(ctas), D1(256), 0, [&] {
    nc::grad_reduce_local_kernel(grad, static_cast<const __nv_bfloat16*>(recv), recv_stride, world, my_rank,
                                 reinterpret_cast<const nc::OwnSeg*>(segs), nsegs, nvec, scale, flags, slot, value, sumsq,
                                 status);
  });
}

void nc_emu_adamw_push(float* master, const long long* value_ptrs, int world, long long value_offset, const float* grad,
                       float* m, float* v, long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                       int step, const float* grad_scale, int ctas) {
  const nc::PeerPtrs values = Peers(value_ptrs, world);
  const float bias1 = 1.0f - std::pow(beta1, static_cast<float>(step));
  const float bias2 = 1.0f - std::pow(beta2, static_cast<float>(step));
  emu::launch(D1(ctas), D1(256), 0, [&] {
    nc::adamw_push_kernel(master, values, value_offset, world, grad, m, v, n, lr, beta1, beta2, eps, weight_decay,
                          1.0f / bias2, lr / bias1, grad_scale);
  });
}

// The Muon update of a shape group with the new bf16 parameters stored into every rank's parameter buffer
// (value_offsets: element offset of each matrix in those buffers).
void nc_emu_muon_apply_push_batched(const long long* master_ptrs, const long long* value_offsets,
                                    const long long* value_ptrs, int world, const void* xb, const float* scale0,
                                    const float* line_scale, int lines_are_rows, int P, int rows, int cols, float lr,
                                    float weight_decay, int ctas) {
  const nc::PeerPtrs values = Peers(value_ptrs, world);
  emu::launch(emu::Dim{static_cast<unsigned>(ctas), static_cast<unsigned>(P), 1}, D1(256), 0, [&] {
    nc::muon_apply_push_batched_kernel(master_ptrs, value_offsets, values, world,
                                       static_cast<const __nv_bfloat16*>(xb), scale0, line_scale, lines_are_rows != 0,
                                       rows, cols, lr, weight_decay);
  });
}

}  // extern "C"

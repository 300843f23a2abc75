// Entry points (C ABI, for ctypes) that run kernels of csrc/cuda on the host through cuda_emu.h. This file includes
// the kernel sources themselves: what runs here is the code the device runs.
#define NC_EMU
#include "../cuda/rowops.cu"

namespace nc {
namespace {
emu::Dim Grid1(long long blocks) { return emu::Dim{static_cast<unsigned>(blocks), 1, 1}; }
emu::Dim Block1(int threads) { return emu::Dim{static_cast<unsigned>(threads), 1, 1}; }
bf16* B(void* p) { return static_cast<bf16*>(p); }
const bf16* B(const void* p) { return static_cast<const bf16*>(p); }
}  // namespace
}  // namespace nc

using nc::B;

extern "C" {

// mode 0: y = norm(x), rstd saved. mode 2: xr = lam_r x + lam_0 x0, y = norm(xr).
void nc_emu_rmsnorm(int mode, const void* x, const void* x0, const float* lam_r, const float* lam_0, void* xr, void* y,
                    float* rstd, int rows, int dim, float eps) {
  const auto grid = nc::Grid1(nc::blocks_for_rows(rows));
  if (mode == 0)
    emu::launch(grid, nc::Block1(nc::kThreads), 0, [&] {
      nc::rmsnorm_kernel<0>(B(x), dim, nullptr, nullptr, nullptr, nullptr, B(y), rstd, rows, dim, eps);
    });
  else
    emu::launch(grid, nc::Block1(nc::kThreads), 0, [&] {
      nc::rmsnorm_kernel<2>(B(x), dim, B(x0), lam_r, lam_0, B(xr), B(y), rstd, rows, dim, eps);
    });
}

void nc_emu_rmsnorm_bwd(const void* x, const void* dy, const float* rstd, const void* residual, void* dx, int rows,
                        int dim) {
  emu::launch(nc::Grid1(nc::blocks_for_rows(rows)), nc::Block1(nc::kThreads), 0,
              [&] { nc::rmsnorm_bwd_kernel(B(x), B(dy), rstd, B(residual), B(dx), rows, dim); });
}

void nc_emu_norm_blend_bwd(const void* xr, const void* dh, const float* rstd, const void* residual, const float* extra,
                           int extra_cols, const void* x, const void* x0, const float* lam_r, const float* lam_0,
                           void* dx, void* dx0, int accumulate, float* g_lam_r, float* g_lam_0, int rows, int dim) {
  emu::launch(nc::Grid1(nc::blocks_for_rows(rows)), nc::Block1(nc::kThreads), 0, [&] {
    nc::norm_blend_bwd_kernel(B(xr), B(dh), rstd, B(residual), extra, extra_cols, B(x), B(x0), lam_r, lam_0, B(dx),
                              B(dx0), accumulate, g_lam_r, g_lam_0, rows, dim);
  });
}

void nc_emu_qk_prep_fwd(const void* in, long long ld_in, void* out, long long ld_out, const float* cosT,
                        const float* sinT, const int* positions, int tokens, int seq, int heads, int D, float eps,
                        float scale) {
  emu::launch(nc::Grid1(nc::blocks_for_rows(tokens)), nc::Block1(nc::kThreads), 0, [&] {
    nc::qk_prep_fwd_kernel(B(in), ld_in, B(out), ld_out, cosT, sinT, positions, tokens, seq, heads, D, eps, scale);
  });
}

void nc_emu_embedding_fwd(const int* ids, const void* table, void* out, int tokens, int dim, int rows, int* status) {
  emu::launch(nc::Grid1(nc::blocks_for_rows(tokens)), nc::Block1(nc::kThreads), 0,
              [&] { nc::embedding_fwd_kernel(ids, B(table), B(out), tokens, dim, rows, status); });
}

void nc_emu_embedding_bwd(const int* ids, const void* dout, long long ld, float* dtable, int tokens, int dim, int rows,
                          int* status) {
  emu::launch(nc::Grid1(nc::blocks_for_rows(tokens)), nc::Block1(nc::kThreads), 0,
              [&] { nc::embedding_bwd_kernel(ids, B(dout), ld, dtable, tokens, dim, rows, status); });
}

void nc_emu_embedding_bwd_sorted(const int* sorted_ids, const int* perm, const void* dout, long long ld, float* dtable,
                                 int tokens, int dim, int rows, int* status) {
  emu::launch(nc::Grid1(nc::blocks_for_rows(tokens)), nc::Block1(nc::kThreads), 0, [&] {
    nc::embedding_bwd_sorted_kernel(sorted_ids, perm, B(dout), ld, dtable, tokens, dim, rows, status);
  });
}

// v += gate * ve (in place), gate saved; with `ids` the value embedding rows are gathered from `ve` as a table.
void nc_emu_value_gate_fwd(const void* h, long long ldh, const void* ve, const void* gate_w, void* v, long long ldv,
                           void* gate, int tokens, int KV, int D, const int* ids, int rows, int* status) {
  const long long pairs = (static_cast<long long>(tokens) * KV + 1) / 2;
  emu::launch(nc::Grid1(nc::blocks_for_rows(pairs)), nc::Block1(nc::kThreads), 0, [&] {
    nc::value_gate_fwd_vec_kernel(B(h), ldh, B(ve), B(gate_w), B(v), ldv, B(gate), tokens, KV, D, ids, rows, status);
  });
}

void nc_emu_value_gate_bwd(const void* h, long long ldh, const void* ve, const void* gate_w, const void* gate,
                           const void* dv, long long lddv, void* dve, float* dh12, float* dgw, int tokens, int KV,
                           int D) {
  emu::launch(nc::Grid1(nc::blocks_for_rows(tokens)), nc::Block1(nc::kThreads), KV * nc::kGateCh * sizeof(float), [&] {
    nc::value_gate_bwd_vec_kernel(B(h), ldh, B(ve), B(gate_w), B(gate), B(dv), lddv, B(dve), dh12, dgw, tokens, KV, D);
  });
}

void nc_emu_smear_fwd(const void* emb, const void* gate_w, const float* lam, const void* prev, void* x0, float* sig,
                      int tokens, int seq, int dim) {
  emu::launch(nc::Grid1(nc::blocks_for_rows(tokens)), nc::Block1(nc::kThreads), 0,
              [&] { nc::smear_fwd_kernel(B(emb), B(gate_w), lam, B(prev), B(x0), sig, tokens, seq, dim); });
}

void nc_emu_qk_prep_bwd(const void* pre, long long ld_pre, const void* grad, long long ld_grad, void* out,
                        long long ld_out, const float* cosT, const float* sinT, int tokens, int seq, int heads, int D,
                        float eps, float scale) {
  emu::launch(nc::Grid1(nc::blocks_for_rows(tokens)), nc::Block1(nc::kThreads), 0, [&] {
    nc::qk_prep_bwd_kernel(B(pre), ld_pre, B(grad), ld_grad, B(out), ld_out, cosT, sinT, tokens, seq, heads, D, eps,
                           scale);
  });
}

// Softcap + cross entropy over bf16 logits, in place (the generic kernel: one block of 256 threads per row).
void nc_emu_classifier(void* logits, long long ld, const int* targets, float* losses, const float* row_scale,
                       const float* dlogit_scale, int rows, int vocab, int padded, float softcap, int ignore_index,
                       int want_grad, int* status) {
  emu::launch(nc::Grid1(rows), nc::Block1(256), 0, [&] {
    nc::classifier_kernel(B(logits), ld, targets, losses, row_scale, dlogit_scale, rows, vocab, padded, softcap,
                          ignore_index, want_grad != 0, status);
  });
}

// The kernel the training step uses by default: 512 threads per row, 16-byte accesses, fixed-cap maximum. `stage`
// parks the row in dynamic shared memory between the two sweeps; stage 2 is the variant that caches exp(z - cap) in place.
void nc_emu_classifier_smem(int stage, void* logits, long long ld, const int* targets, float* losses,
                            const float* row_scale, const float* dlogit_scale, int rows, int vocab, int padded,
                            float softcap, int ignore_index, int want_grad, int* status) {
  if (stage == 2)
    emu::launch(nc::Grid1(rows), nc::Block1(nc::kClsThreads), 0, [&] {
      nc::classifier_smem_kernel<false, true>(B(logits), ld, targets, losses, row_scale, dlogit_scale, vocab, padded,
                                              softcap, ignore_index, want_grad != 0, status);
    });
  else if (stage)
    emu::launch(nc::Grid1(rows), nc::Block1(nc::kClsThreads), want_grad ? static_cast<size_t>(padded) * 2 : 0, [&] {
      nc::classifier_smem_kernel<true>(B(logits), ld, targets, losses, row_scale, dlogit_scale, vocab, padded, softcap,
                                       ignore_index, want_grad != 0, status);
    });
  else
    emu::launch(nc::Grid1(rows), nc::Block1(nc::kClsThreads), 0, [&] {
      nc::classifier_smem_kernel<false>(B(logits), ld, targets, losses, row_scale, dlogit_scale, vocab, padded, softcap,
                                        ignore_index, want_grad != 0, status);
    });
}

void nc_emu_smear_bwd(const void* emb, const void* gate_w, const float* lam, const float* sig, const void* dx0, void* de,
                      float* dgw24, float* dlam, int tokens, int seq, int dim) {
  emu::launch(nc::Grid1(nc::blocks_for_rows(tokens)), nc::Block1(nc::kThreads), 0, [&] {
    nc::smear_bwd_kernel(B(emb), B(gate_w), lam, sig, B(dx0), B(de), dgw24, dlam, tokens, seq, dim);
  });
}

// Gradient norm over several fp32 spans: one sum-of-squares launch per span into one fp64 accumulator, then the
// norm and the clip factor (out2[0], out2[1]).
void nc_emu_grad_norm(const long long* spans, const long long* lengths, int count, double* acc, float clip, float* out2,
                      int blocks) {
  *acc = 0.0;
  for (int i = 0; i < count; ++i)
    emu::launch(nc::Grid1(blocks), nc::Block1(256), 0,
                [&] { nc::sumsq_kernel(reinterpret_cast<const float*>(spans[i]), lengths[i], acc); });
  emu::launch(nc::Grid1(1), nc::Block1(1), 0, [&] { nc::finish_norm_kernel(acc, clip, out2); });
}

void nc_emu_add_cols(void* dh, long long ld, const float* extra, int rows, int ncols) {
  emu::launch(nc::Grid1((rows * ncols + 255) / 256), nc::Block1(256), 0,
              [&] { nc::add_cols_kernel(B(dh), ld, extra, rows, ncols); });
}

// Self-test of the scheduler: 64 threads write their index in the order in which they first run, then meet at a
// barrier and write it again in the order in which they leave it.
void nc_emu_selftest_order(int* first_run, int* after_barrier) {
  int n1 = 0, n2 = 0;
  emu::launch(nc::Grid1(1), nc::Block1(64), 0, [&] {
    first_run[n1++] = static_cast<int>(threadIdx.x);
    __syncthreads();
    after_barrier[n2++] = static_cast<int>(threadIdx.x);
  });
}

}  // extern "C"

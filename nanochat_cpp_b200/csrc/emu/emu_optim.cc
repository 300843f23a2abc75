// Host entry points for the optimizer kernels (csrc/cuda/optim.cu compiled over cuda_emu.h).
#define NC_EMU
#include "../cuda/optim.cu"

#include <cmath>

extern "C" {

// One AdamW step on n elements, as `nc::adamw_update` launches it (value: bf16 copy, may be null).
void nc_emu_adamw(float* master, void* value, const float* grad, float* m, float* v, long long n, float lr, float beta1,
                  float beta2, float eps, float weight_decay, int step, const float* grad_scale, int blocks) {
  const float bias1 = 1.0f - std::pow(beta1, static_cast<float>(step));
  const float bias2 = 1.0f - std::pow(beta2, static_cast<float>(step));
  emu::launch(emu::Dim{static_cast<unsigned>(blocks), 1, 1}, emu::Dim{256, 1, 1}, 0, [&] {
    nc::adamw_kernel(master, static_cast<__nv_bfloat16*>(value), grad, m, v, n, lr, beta1, beta2, eps, weight_decay,
                     1.0f / bias2, lr / bias1, grad_scale);
  });
}

// x = Nesterov(grad, buf1) and per-row sums of squares (first Muon stage).
void nc_emu_muon_nesterov(const float* grad, float* buf1, float* x, float* row_sumsq, int rows, int cols, float momentum,
                          const float* grad_scale) {
  emu::launch(emu::Dim{static_cast<unsigned>((rows + 7) / 8), 1, 1}, emu::Dim{256, 1, 1}, 0,
              [&] { nc::muon_nesterov_kernel(grad, buf1, x, row_sumsq, rows, cols, momentum, grad_scale); });
}

// The element-wise stages of a batched Muon step for one shape group, in the order optim/muon_cuda.py launches them,
// with the Newton-Schulz products left out (X passes from the first half to the second unchanged): momentum and
// row sums, equilibration scales, scaled bf16 X, line sums of squares, Muon+ / NorMuon statistics, update.
void nc_emu_muon_group_no_ns(const long long* grad_ptrs, const long long* buf1_ptrs, const long long* buf2_ptrs,
                             const long long* master_ptrs, const long long* value_ptrs, float* x32, float* row_ss,
                             float* row_scale, float* all_scale, void* X, float* line_ss, float* scale,
                             float* line_scale, int P, int rows, int cols, float momentum, float beta2, float lr,
                             float weight_decay, const float* grad_scale) {
  using bf = __nv_bfloat16;
  const unsigned up = static_cast<unsigned>(P);
  const emu::Dim by_rows{static_cast<unsigned>((rows + 7) / 8), up, 1}, b256{256, 1, 1};
  const bool reduce_cols = rows >= cols;
  const int lines = reduce_cols ? rows : cols, line_len = reduce_cols ? cols : rows;
  emu::launch(by_rows, b256, 0, [&] {
    nc::muon_nesterov_batched_kernel(grad_ptrs, buf1_ptrs, x32, row_ss, rows, cols, momentum, grad_scale);
  });
  emu::launch(emu::Dim{up, 1, 1}, b256, 0, [&] { nc::muon_prescale_kernel(row_ss, row_scale, all_scale, rows); });
  emu::launch(by_rows, b256, 0, [&] {
    nc::muon_scale_rows_batched_kernel(x32, row_scale, all_scale, static_cast<bf*>(X), rows, cols);
  });
  const emu::Dim line_grid = reduce_cols ? by_rows : emu::Dim{static_cast<unsigned>((cols / 2 + 255) / 256), up, 1};
  emu::launch(line_grid, b256, 0,
              [&] { nc::muon_line_sumsq_kernel(static_cast<const bf*>(X), line_ss, rows, cols, reduce_cols); });
  emu::launch(emu::Dim{up, 1, 1}, b256, 0, [&] {
    nc::muon_poststats_kernel(line_ss, buf2_ptrs, scale, line_scale, lines, line_len,
                              std::sqrt(static_cast<float>(rows < cols ? rows : cols)), beta2);
  });
  long long blocks = (static_cast<long long>(rows) * cols / 2 + 255) / 256;
  if (blocks > 16) blocks = 16;  // grid-stride loop: fewer blocks than the device launch, same coverage
  emu::launch(emu::Dim{static_cast<unsigned>(blocks), up, 1}, b256, 0, [&] {
    nc::muon_apply_batched_kernel(master_ptrs, value_ptrs, static_cast<const bf*>(X), scale, line_scale, reduce_cols,
                                  rows, cols, lr, weight_decay);
  });
}

void nc_emu_relu2(const void* x, void* y, long long n, int blocks) {
  emu::launch(emu::Dim{static_cast<unsigned>(blocks), 1, 1}, emu::Dim{256, 1, 1}, 0, [&] {
    nc::relu2_kernel(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n);
  });
}

void nc_emu_cast(const float* x, void* y, long long n, int blocks) {
  emu::launch(emu::Dim{static_cast<unsigned>(blocks), 1, 1}, emu::Dim{256, 1, 1}, 0,
              [&] { nc::cast_kernel(x, static_cast<__nv_bfloat16*>(y), n); });
}

void nc_emu_muon_apply_batched(const long long* master_ptrs, const long long* value_ptrs, const void* xb,
                               const float* scale0, const float* line_scale, int lines_are_rows, int P, int rows,
                               int cols, float lr, float weight_decay, int ctas) {
  emu::launch(emu::Dim{static_cast<unsigned>(ctas), static_cast<unsigned>(P), 1}, emu::Dim{256, 1, 1}, 0, [&] {
    nc::muon_apply_batched_kernel(master_ptrs, value_ptrs, static_cast<const __nv_bfloat16*>(xb), scale0, line_scale,
                                  lines_are_rows != 0, rows, cols, lr, weight_decay);
  });
}

// The one-launch Muon step of P small matrices. coeffs: 15 floats, five (a, b, c) triples.
void nc_emu_muon_tiny(const long long* grad_ptrs, const long long* buf1_ptrs, const long long* buf2_ptrs,
                      const long long* master_ptrs, const long long* value_ptrs, int P, int rows, int cols,
                      float momentum, float beta2, float lr, float weight_decay, int ns_steps, const float* grad_scale,
                      const float* coeffs) {
  nc::TinyCoeffs c;
  for (int i = 0; i < 5; ++i)
    for (int j = 0; j < 3; ++j) c.c[i][j] = coeffs[i * 3 + j];
  emu::launch(emu::Dim{static_cast<unsigned>(P), 1, 1}, emu::Dim{128, 1, 1}, 0, [&] {
    nc::muon_tiny_kernel(grad_ptrs, buf1_ptrs, buf2_ptrs, master_ptrs, value_ptrs, rows, cols, momentum, beta2, lr,
                         weight_decay, ns_steps, grad_scale, c);
  });
}

}  // extern "C"

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

}  // extern "C"

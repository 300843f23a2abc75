// Host launchers of the optimizer kernels (optim.cu). fp32 state, bf16 compute copies.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace nc {

// Decoupled-decay AdamW on an fp32 master span; writes the bf16 compute copy when `value` != null.
// `grad_scale` is a device scalar (the clip scale). Arithmetic: reference backends/cpu/kernels.cc:1557-1580.
void adamw_update(float* master, __nv_bfloat16* value, const float* grad, float* m, float* v, long long n, float lr,
                  float beta1, float beta2, float eps, float weight_decay, int step, const float* grad_scale,
                  cudaStream_t s);

// Muon stage 1 for one matrix [rows, cols]: buf1 += (1-mu)(g*scale - buf1); x = (1-mu) g*scale + mu*buf1;
// row_sumsq[r] = sum_c x[r,c]^2.
void muon_nesterov(const float* grad, float* buf1, float* x, float* row_sumsq, int rows, int cols, float momentum,
                   const float* grad_scale, cudaStream_t s);
// x[r,:] *= row_scale[r] * all_scale[0]; out bf16 copy; also out_sumsq (optional, double) of the scaled matrix
void muon_scale_rows(const float* x, const float* row_scale, const float* all_scale, __nv_bfloat16* out, int rows,
                     int cols, cudaStream_t s);
// Cautious decay + update: p -= lr*x*line_scale + (x*p >= 0 ? lr*wd*p : 0), x = xb * scale[0] * line_scale[line].
void muon_apply(float* master, __nv_bfloat16* value, const __nv_bfloat16* xb, const float* scale0,
                const float* line_scale, bool lines_are_rows, int rows, int cols, float lr, float weight_decay,
                cudaStream_t s);
// Batched forms over the P matrices [rows, cols] of a shape group (cols a multiple of 8). Pointer tables are device
// arrays of P addresses; x, row_sumsq, xb, scale0, line_scale are stacked [P, ...] tensors.
void muon_nesterov_batched(const long long* grad_ptrs, const long long* buf1_ptrs, float* x, float* row_sumsq, int P,
                           int rows, int cols, float momentum, const float* grad_scale, cudaStream_t s);
void muon_scale_rows_batched(const float* x, const float* row_scale, const float* all_scale, __nv_bfloat16* out, int P,
                             int rows, int cols, cudaStream_t s);
void muon_line_sumsq(const __nv_bfloat16* x, float* out, int P, int rows, int cols, bool reduce_cols, cudaStream_t s);
// One CTA per matrix: row_ss [P, rows] -> row_scale [P, rows], all_scale [P] (row equilibration + normalisation).
void muon_prescale(const float* row_ss, float* row_scale, float* all_scale, int P, int rows, cudaStream_t s);
// One CTA per matrix: line_ss [P, lines] + NorMuon state (table of per-matrix buf2 addresses) -> scale [P],
// line_scale [P, lines]; updates buf2 in place. `target_norm` = sqrt(min(rows, cols)).
void muon_poststats(const float* line_ss, const long long* buf2_ptrs, float* scale_out, float* line_scale, int P,
                    int lines, int line_len, float target_norm, float beta2, cudaStream_t s);
void muon_apply_batched(const long long* master_ptrs, const long long* value_ptrs, const __nv_bfloat16* xb,
                        const float* scale0, const float* line_scale, bool lines_are_rows, int P, int rows, int cols,
                        float lr, float weight_decay, cudaStream_t s);
// relu(x)^2 elementwise (bf16)
// Whole Muon step of P small matrices (rows * cols <= 1024, smaller side <= 32) given by pointer tables, one launch.
// coeffs: the five (a, b, c) triples of the Polar Express iteration. Returns an error text for a shape it does not take.
const char* muon_tiny(const long long* grad_ptrs, const long long* buf1_ptrs, const long long* buf2_ptrs,
                      const long long* master_ptrs, const long long* value_ptrs, int P, int rows, int cols, float momentum,
                      float beta2, float lr, float weight_decay, int ns_steps, const float* grad_scale,
                      const double (*coeffs)[3], cudaStream_t s);

void relu2_bf16(const __nv_bfloat16* x, __nv_bfloat16* y, long long n, cudaStream_t s);
// bf16 <- fp32 cast of a span
void cast_f32_bf16(const float* x, __nv_bfloat16* y, long long n, cudaStream_t s);

}  // namespace nc

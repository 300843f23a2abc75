// Host launchers of the memory-bound row kernels (rowops.cu). All activations are bf16, all
// statistics and parameter gradients fp32. `ld*` are row strides in elements. Every launcher enqueues
// on `stream` and returns immediately.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nc {

using bf16 = __nv_bfloat16;

// y = x * rsqrt(mean(x^2) + eps); rstd saved per row.
// With `yq` and `sf` the kernel also writes y as MXFP8 (E4M3 codes [rows, dim] + scale atoms for 128-row tiles, the
// layout of fp8.h); needs dim % 128 == 0 and 16-byte aligned rows.
void rmsnorm_fwd(const bf16* x, long long ldx, bf16* y, float* rstd, int rows, int dim, float eps, cudaStream_t s,
                 uint8_t* yq = nullptr, uint8_t* sf = nullptr);
void rmsnorm_apply(const bf16* x, long long ldx, const float* rstd, bf16* y, int rows, int dim, cudaStream_t s);
// dx = rstd*dy - rstd^3 * mean(x*dy) * x (+ residual)
void rmsnorm_bwd(const bf16* x, const bf16* dy, const float* rstd, const bf16* residual, bf16* dx, int rows, int dim,
                 cudaStream_t s);
// xr = lam_r*x + lam_0*x0 ; h = rmsnorm(xr)
void blend_norm_fwd(const bf16* x, const bf16* x0, const float* lam_r, const float* lam_0, bf16* xr, bf16* h,
                    float* rstd, int rows, int dim, float eps, cudaStream_t s, uint8_t* hq = nullptr,
                    uint8_t* sf = nullptr);
// dx = lam_r*dxr ; dx0 (+)= lam_0*dxr ; dlam[0] += <dxr,x> ; dlam[1] += <dxr,x0>
// rmsnorm backward + blend backward in one pass (see the kernel): dxr stays in registers; the two scalar gradients are
// added into g_lam_r / g_lam_0 (device scalars inside the flat gradient); `extra` [rows, extra_cols] fp32 is added to
// the first columns of dh first (may be null). Returns an error string for shapes it does not take.
const char* norm_blend_bwd(const bf16* xr, const bf16* dh, const float* rstd, const bf16* residual, const float* extra,
                           int extra_cols, const bf16* x, const bf16* x0, const float* lam_r, const float* lam_0, bf16* dx,
                           bf16* dx0, bool accumulate_dx0, float* g_lam_r, float* g_lam_0, int rows, int dim,
                           cudaStream_t s);
void blend_bwd(const bf16* dxr, const bf16* x, const bf16* x0, const float* lam_r, const float* lam_0, bf16* dx,
               bf16* dx0, bool accumulate_dx0, float* dlam2, long long n, cudaStream_t s);
// y = x - lam*xb
void backout_fwd(const bf16* x, const bf16* xb, const float* lam, bf16* y, long long n, cudaStream_t s);
// dxb = -lam*dy ; dlam[0] += -<dy, xb>
void backout_bwd(const bf16* dy, const bf16* xb, const float* lam, bf16* dxb, float* dlam, long long n,
                 cudaStream_t s);
void add_bf16(const bf16* a, const bf16* b, bf16* out, long long n, cudaStream_t s);
// dh[:, :ncols] += extra (fp32 [rows, ncols])
void add_cols(bf16* dh, long long ld, const float* extra, int rows, int ncols, cudaStream_t s);

// Per-head RMSNorm -> RoPE (half split) -> scale. in: [tokens, heads, D] with token stride ld_in; out contiguous.
// pos[token] = position inside its sequence = token % seq (or explicit positions when `positions` != null).
void qk_prep_fwd(const bf16* in, long long ld_in, bf16* out, long long ld_out, const float* cos, const float* sin,
                 const int* positions, int tokens, int seq, int heads, int D, float eps, float scale, cudaStream_t s);
void qk_prep_bwd(const bf16* pre, long long ld_pre, const bf16* grad, long long ld_grad, bf16* out, long long ld_out,
                 const float* cos, const float* sin, int tokens, int seq, int heads, int D, float eps, float scale,
                 cudaStream_t s);

// v += 3*sigmoid(h[:, :12] . w[kh]) * ve  (in place on v); gate saved as bf16 [tokens, KV]
void value_gate_fwd(const bf16* h, long long ldh, const bf16* ve, const bf16* gate_w, bf16* v, long long ldv,
                    bf16* gate, int tokens, int KV, int D, cudaStream_t s,
                    const int* ids = nullptr, int rows = 0, int* status = nullptr);
// ids: `ve` is an embedding table [vocab, KV * D], row ids[tok] is used
void value_gate_bwd(const bf16* h, long long ldh, const bf16* ve, const bf16* gate_w, const bf16* gate, const bf16* dv,
                    long long lddv, bf16* dve, float* dh12, float* dgw, int tokens, int KV, int D, cudaStream_t s);

// x[t] = e[t] + lam*sigmoid(e[t,:24].w)*e[t-1]; first row of every sequence uses `prev` (or nothing).
void smear_fwd(const bf16* emb, const bf16* gate_w, const float* lam, const bf16* prev, bf16* x0, float* sig,
               int tokens, int seq, int dim, cudaStream_t s);
void smear_bwd(const bf16* emb, const bf16* gate_w, const float* lam, const float* sig, const bf16* dx0, bf16* de,
               float* dgw24, float* dlam, int tokens, int seq, int dim, cudaStream_t s);

// `rows` > 0: the table's row count; an id outside it is skipped (forward: a zero row) and `status` gets kErrBadIndex.
void embedding_fwd(const int* ids, const bf16* table, bf16* out, int tokens, int dim, cudaStream_t s, int rows = 0,
                   int* status = nullptr);
// dtable[ids[t]] += dout[t] (fp32 accumulate, vector red.global.add)
void embedding_bwd(const int* ids, const bf16* dout, long long ld, float* dtable, int tokens, int dim, cudaStream_t s,
                   int rows = 0, int* status = nullptr);
// Same sum with a fixed order: `sorted_ids` stably sorted, `perm` the original row of each sorted position.
void embedding_bwd_sorted(const int* sorted_ids, const int* perm, const bf16* dout, long long ld, float* dtable,
                          int tokens, int dim, cudaStream_t s, int rows = 0, int* status = nullptr);

// Softcap + cross entropy over [rows, padded] bf16 logits, in place: logits are overwritten by dlogits when
// `want_grad`. dlogit_scale is a device scalar. losses[row] = 0 on ignored rows.
void classifier_fwd_bwd(bf16* logits, long long ld, const int* targets, float* losses, const float* row_scale,
                        const float* dlogit_scale, int rows, int vocab, int padded, float softcap, int ignore_index,
                        bool want_grad, cudaStream_t s, int* status = nullptr);
// A target outside [0, vocab) other than `ignore_index` counts as ignored and records kErrBadIndex in `status`.

// sum of squares of an fp32 span, accumulated into out[0] (double)
void sumsq_f32(const float* g, long long n, double* out, cudaStream_t s);
// norm_clip[0] = sqrt(sumsq), norm_clip[1] = clip scale
void finish_norm(const double* sumsq, float clip, float* norm_clip, cudaStream_t s);

}  // namespace nc

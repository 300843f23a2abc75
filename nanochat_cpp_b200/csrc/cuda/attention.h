// Host interface of the flash-attention kernels (attention_fwd.cu, attention_bwd.cu).
// Tensors are bf16 views of token-major activations: element (b, t, h, d) at
// ptr[b*stride_b + t*stride_t + h*stride_h + d]; strides in elements, all multiples of 8.
#pragma once
#include <cuda_runtime.h>

namespace nc {

struct AttnArgs {
  int B = 0, H = 0, KVH = 0, Tq = 0, Tk = 0, D = 0;
  int q_offset = 0;      // absolute position of query row 0 (Tk - Tq during training)
  int window_left = -1;  // < 0: full causal context
  float scale = 1.0f;
  const void *Q = nullptr, *K = nullptr, *V = nullptr;
  long long q_stride_b = 0, q_stride_t = 0, q_stride_h = 0;
  long long k_stride_b = 0, k_stride_t = 0, k_stride_h = 0;
  long long v_stride_b = 0, v_stride_t = 0, v_stride_h = 0;
  void* O = nullptr;
  long long o_stride_b = 0, o_stride_t = 0, o_stride_h = 0;
  float* lse = nullptr;  // [B, H, Tq]
  // backward only
  const void* dO = nullptr;
  long long do_stride_b = 0, do_stride_t = 0, do_stride_h = 0;
  float* delta = nullptr;  // [B, H, Tq] scratch: rowsum(dO * O)
  // Optional scratch for dS^T [B, H, ds_tk, ds_tq] bf16 (ds_tk = Tk rounded up to 128, ds_tq = Tq rounded up to
  // 128). When given, the dK/dV kernel stores the dS tiles it computes and dQ = dS K runs as a banded GEMM over
  // them (attention_dq.cu) instead of recomputing scores and probabilities.
  void* dS = nullptr;
  long long ds_tk = 0, ds_tq = 0;
  void *dQ = nullptr, *dK = nullptr, *dV = nullptr;
  long long dq_stride_b = 0, dq_stride_t = 0, dq_stride_h = 0;
  long long dk_stride_b = 0, dk_stride_t = 0, dk_stride_h = 0;
  long long dv_stride_b = 0, dv_stride_t = 0, dv_stride_h = 0;
  int* status = nullptr;
};

// one 128-row query tile per CTA, running output in registers
const char* attention_fwd(const AttnArgs& args, cudaStream_t stream);
// two query tiles per CTA, running output in TMEM with lazy rescaling (the default)
const char* attention_fwd2(const AttnArgs& args, cudaStream_t stream);
const char* attention_bwd(const AttnArgs& args, cudaStream_t stream);
// dQ from stored dS^T (used by attention_bwd when AttnArgs::dS is set)
const char* attention_dq_from_ds(const AttnArgs& args, cudaStream_t stream);

}  // namespace nc

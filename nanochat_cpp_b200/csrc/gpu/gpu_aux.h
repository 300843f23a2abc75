// Small device helpers of the C++ GPU engine that have no counterpart among the model kernels.
#pragma once
#include <cuda_runtime.h>

namespace ncb {

// resid_grad[i] += pairs[2 i], x0_grad[i] += pairs[2 i + 1] for i < layers (the per-layer scalar gradients that the
// blend backward accumulated in a scratch array).
void gpu_scatter_pairs_add(float* resid_grad, float* x0_grad, const float* pairs, int layers, cudaStream_t s);

}  // namespace ncb

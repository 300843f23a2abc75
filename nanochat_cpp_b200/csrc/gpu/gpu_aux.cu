#include "gpu_aux.h"

namespace ncb {

namespace {
__global__ void scatter_pairs_add_kernel(float* resid_grad, float* x0_grad, const float* pairs, int layers) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < layers) {
    resid_grad[i] += pairs[2 * i];
    x0_grad[i] += pairs[2 * i + 1];
  }
}
}  // namespace

void gpu_scatter_pairs_add(float* resid_grad, float* x0_grad, const float* pairs, int layers, cudaStream_t s) {
  if (layers > 0) scatter_pairs_add_kernel<<<(layers + 127) / 128, 128, 0, s>>>(resid_grad, x0_grad, pairs, layers);
}

}  // namespace ncb

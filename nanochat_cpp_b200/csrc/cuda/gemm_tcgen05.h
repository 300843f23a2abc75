// Host interface of the tcgen05 bf16 GEMM (gemm_tcgen05.cu).
#pragma once
#include <cuda_runtime.h>

namespace nc {

enum GemmEpilogue : int {
  kEpiBf16 = 0,     // C = bf16(alpha * acc)
  kEpiBf16Res = 1,  // C = bf16(alpha * acc + beta * R)                  (R bf16, same shape as C)
  kEpiRelu2 = 2,    // C = bf16(acc); C2 = bf16(relu(C)^2)               (MLP up-projection)
  kEpiDRelu2 = 3,   // C = bf16(acc * 2 * relu(R))                       (backward of relu^2; R = pre-activation)
  kEpiF32 = 4,      // C32 = alpha * acc + beta * C32                    (weight gradients; may split K)
};

struct GemmArgs {
  // C[b][M,N] = sum_k A[b][m,k] * B[b][n,k].
  // K-major operand:  element (row, k) at ptr[row * ld + k].
  // MN-major operand: element (row, k) at ptr[k * ld + row].
  const void* A = nullptr;
  const void* B = nullptr;
  long long lda = 0, ldb = 0;
  bool a_mn_major = false, b_mn_major = false;
  int M = 0, N = 0, K = 0;
  int batch = 1;
  long long strideA = 0, strideB = 0, strideC = 0, strideR = 0;  // elements, between batches
  void* C = nullptr;
  long long ldc = 0;
  void* C2 = nullptr;        // kEpiRelu2 second output, same ld/stride as C
  const void* R = nullptr;   // kEpiBf16Res / kEpiDRelu2
  long long ldr = 0;
  float alpha = 1.0f, beta = 0.0f;
  int epi = kEpiBf16;
  bool allow_split_k = true;  // kEpiF32 only: split K across CTAs when there are fewer tiles than SMs
  int* status = nullptr;      // device status word (see ptx.cuh error codes); may be null
};

// Returns nullptr on success or a static error string.
const char* gemm_bf16(const GemmArgs& args, cudaStream_t stream);

}  // namespace nc

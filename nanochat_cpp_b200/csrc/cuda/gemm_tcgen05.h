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
  // Data-parallel hooks for the B operand (the weight), both optional:
  //  * wait_flags: the TMA producer does not touch B before wait_flags[i] >= wait_value for all i < wait_count
  //    (owners publish these flags after pushing updated weights into this rank's parameter buffer);
  //  * gather_src: B is first copied from `gather_src` (a peer mapping of the owner's copy) into its local
  //    address by all CTAs (plain peer loads), then a grid-wide counter releases the TMA producers. The
  //    tensor map always points at local memory. gather_counter must count up monotonically across calls:
  //    pass the value it will have reached when every CTA of this launch has arrived (kernel adds grid each call).
  const int* wait_flags = nullptr;
  int wait_count = 0, wait_value = 0;
  const void* gather_src = nullptr;
  long long gather_bytes = 0;
  int* gather_counter = nullptr;
  int gather_base = 0;  // counter value before this launch
};

// Returns nullptr on success or a static error string.
const char* gemm_bf16(const GemmArgs& args, cudaStream_t stream);
// Decode-shaped products (M <= 64, K-major operands, batch 1, epilogues bf16 / bf16+residual / relu^2): weight rows
// on the MMA's M side, K split over a thread-block cluster (gemm_skinny.cu).
const char* gemm_skinny(const GemmArgs& args, cudaStream_t stream);

}  // namespace nc

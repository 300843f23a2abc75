// Link-time stand-ins for the three parts of the reference that cannot be built on this image.
// Nothing here changes what the reference computes on a B200: each stand-in gives the answer the real
// object gives on a device that is not an sm_90a part, or covers a path the benchmark never takes.
//
//  * CUTLASS Sm90 GEMM launchers (backends/cuda/gemm/cutlass_launch.h:39-60 of the reference). The real
//    objects are pinned to sm_90a and refuse every device whose compute capability is not 9.0
//    (backends/cuda/gemm/cutlass_kernel.cuh:127-129) by returning false, after which gemm.cu keeps its
//    hand tile and then cuBLAS. The stand-ins return false unconditionally.
//  * OpenParquetSource (src/parquet/reader.h:56). The parquet reader needs zstd.h, which the image lacks.
//    The harness feeds documents through TrainConfig::train_source, so this is only called when a run
//    names parquet files; it then reports that the reader is absent.
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "nanochat/dataloader.h"
#include "nanochat/kernels.h"
#include "nanochat/tensor.h"

namespace nanochat {

std::unique_ptr<DocumentSource> OpenParquetSource(const std::vector<std::string>&, const std::string&,
                                                  std::size_t, std::string* error) {
  if (error != nullptr) *error = "parquet reader not built (no zstd.h on this image)";
  return nullptr;
}

#if defined(NANOCHAT_REF_CUDA)
namespace kernels {

struct ResolvedGemm;

bool LaunchGemmCutlass(const ResolvedGemm&, const ComputeType*, const ComputeType*, ComputeType*) {
  return false;
}
bool LaunchGemmCutlassToFp32(const ResolvedGemm&, const ComputeType*, const ComputeType*, float*) {
  return false;
}
int GemmCutlassKernelCount() { return 0; }
bool LaunchScaledFp8Cutlass(const ScaledGemmParams&, const std::uint8_t*, const std::uint8_t*, ComputeType*) {
  return false;
}
bool LaunchScaledFp8CutlassToFp32(const ScaledGemmParams&, const std::uint8_t*, const std::uint8_t*, float*) {
  return false;
}
const char* GemmCutlassTileName() { return "absent"; }

}  // namespace kernels
#endif

}  // namespace nanochat

// Launch helper for kernels that call griddepcontrol.wait before their first dependent access: with the process-wide
// switch on (the inference engine turns it on around a decode step) they are launched with programmatic stream
// serialization, so their blocks are already resident and waiting when the previous kernel of the stream ends;
// with the switch off it is an ordinary launch.
#pragma once
#include <cuda_runtime.h>

namespace nc {

bool pdl_enabled();
void set_pdl_enabled(bool on);

template <class... KArgs, class... Args>
inline cudaError_t launch_maybe_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace nc

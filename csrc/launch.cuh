// Kernel launch through cudaLaunchKernelEx with the programmatic-serialization attribute when
// `cosmos::pdl_on()`; a plain launch otherwise. Only for kernels that execute `pdl_wait()` before they touch
// anything a predecessor wrote.
#pragma once
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "kernels.h"

namespace cosmos {

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_on() ? 1 : 0;
  const cudaError_t err = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
  if (err != cudaSuccess) throw std::runtime_error(std::string("kernel launch failed: ") + cudaGetErrorString(err));
}

}  // namespace cosmos

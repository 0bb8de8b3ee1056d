// Kernel launch with programmatic dependent launch (PDL) allowed: the kernel may be scheduled while its predecessor in
// the stream drains, runs its prologue, and waits in griddep_wait() for the predecessor's results.  Only kernels that call
// griddep_wait() before their first access to global memory may be launched this way.  DICE_B200_PDL=0 switches the
// attribute off (the launches are then ordinary stream-ordered launches).
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <utility>

namespace dice {

static inline bool pdl_enabled() {
  static int state = -1;
  if (state < 0) {
    const char* v = std::getenv("DICE_B200_PDL");
    state = (v != nullptr && std::strcmp(v, "0") == 0) ? 0 : 1;
  }
  return state == 1;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(std::forward<Args>(args))...);
}

}  // namespace dice

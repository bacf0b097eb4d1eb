// Launch helper with programmatic dependent launch (PDL): a kernel launched through sfb_launch may be
// scheduled while its stream predecessor is still draining; it runs its set-up code and then blocks in
// pdl_wait() until the predecessor has completed and its writes are visible.  Every kernel launched this
// way calls pdl_wait() before it reads anything a predecessor wrote, and pdl_launch_dependents() early
// so that its own successor can start its set-up.  Inside stream capture these become programmatic
// dependency edges of the graph.  (Reference: kernels/opt_pdl_sm121.cuh - griddepcontrol on the decode chain.)
#pragma once
#include <cuda_runtime.h>

#include <utility>

namespace sfb {

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline int& pdl_enabled() {
  static int on = 1;
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t sfb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace sfb

// Programmatic dependent launch: every kernel of the decode step is launched with the
// programmatic-stream-serialization attribute, calls pdl_launch_dependents() at its start (the next
// kernel's CTAs may become resident as SMs free up) and pdl_wait() before it reads anything an
// earlier kernel wrote or writes anything an earlier kernel may still read.  pdl_wait() returns only
// when the whole prerequisite grid has completed and its memory is visible, and that grid itself
// waited for its own predecessor, so completion is transitive along the stream.  What runs before
// the wait touches immutable data only (weights).  Without the attribute both calls do nothing.
#pragma once
#include <cuda_runtime.h>

namespace lmb {

bool pdl_enabled();
void pdl_set_enabled(bool on);

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// `overlap` = false launches with ordinary stream order (the kernel starts only after its
// predecessor has drained), for kernels that must not share an SM configuration with it.
template <typename... KArgs, typename... Args>
cudaError_t launch_k_opt(bool overlap, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                         Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (overlap && pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  return launch_k_opt(true, kern, grid, block, smem, st, static_cast<Args&&>(args)...);
}

}  // namespace lmb

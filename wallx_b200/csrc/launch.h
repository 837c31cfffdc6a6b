// Programmatic dependent launch for chains of small kernels (decode and denoise steps inside a CUDA graph).
//
// A kernel launched through launch_kernel() while the switch is on may start before the kernel ahead of it in the
// stream has finished: its blocks are scheduled onto free SMs, run their prologue (barrier set-up, tensor-memory
// allocation, descriptor prefetch) and then stop in pdl_wait() until the earlier grid has completed and its writes
// are visible. Every kernel launched this way therefore calls pdl_wait() before its first access to global memory
// that an earlier kernel may have written, and pdl_launch_dependents() once the next kernel may begin its own
// prologue. Both instructions do nothing in a kernel that was launched the ordinary way, and a kernel without
// pdl_wait() is never launched through this helper. The switch is off by default (training launches are unchanged);
// the flow engine turns it on around its graph capture.
#pragma once
#include <cuda_runtime.h>

namespace wx {

bool pdl_enabled();
void pdl_set(bool on);

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// `cluster_x` > 1 launches thread-block clusters of that many CTAs along x (the grid's x must be a multiple of it).
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  unsigned cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  return launch_kernel_cluster(kern, grid, block, smem, stream, 1u, args...);
}
#endif

}  // namespace wx

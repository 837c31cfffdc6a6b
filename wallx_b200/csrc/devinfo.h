// Properties of the current device that size grids (queried once per device, never hard-coded).
#pragma once
#include <cuda_runtime.h>

namespace wx {

// Number of SMs of the current device; grids are sized in resident blocks per SM.
inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 1;
  }
  return cached[dev];
}

}  // namespace wx

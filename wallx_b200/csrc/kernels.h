// Host launchers of the non-GEMM kernels (raw pointers + stream; no torch types).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace wx {}  // namespace wx

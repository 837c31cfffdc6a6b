// Bindings of the non-GEMM kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "kernels.h"

void register_kernel_bindings(pybind11::module_& m) { (void)m; }

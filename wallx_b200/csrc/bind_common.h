// Helpers shared by the binding translation units (torch types -> raw-pointer launch structs).
#pragma once
#include <torch/extension.h>

#include <tuple>
#include <vector>

#include "gemm.h"

namespace wxb {

using OptT = c10::optional<at::Tensor>;

// One GEMM problem as Python hands it over: (A, a_mn, B, b_mn, D, M, N, K, bias, residual, row_map, dyn, D2, flags, m0, k0).
using GemmTuple = std::tuple<at::Tensor, bool, at::Tensor, bool, at::Tensor, int64_t, int64_t, int64_t, OptT, OptT,
                             OptT, OptT, OptT, int64_t, int64_t, int64_t>;

// Throws std::runtime_error with the launch's return code (positive codes are cudaError_t values).
[[noreturn]] void fail_code(const char* what, int rc);

// Per-device int32[4] status words that kernels set when a bounded wait runs out.
at::Tensor& status_tensor(const at::Device& dev);

// Validates the tensors of one problem and fills the launch struct.
void fill_call(wx::GemmCall& c, const GemmTuple& g);

}  // namespace wxb

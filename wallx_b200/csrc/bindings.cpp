// Python bindings (torch tensors -> raw-pointer launchers). This is the only translation unit
// that sees torch headers; the kernels live in plain .cu files.
//
// Reference parity: csrc/ops.cu:11-21 (the pybind table of the reference's nine ops).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <tuple>
#include <vector>

#include "gemm.h"
#include "kernels.h"

namespace {

using OptT = c10::optional<at::Tensor>;

at::Tensor& status_tensor(const at::Device& dev) {
  static std::vector<at::Tensor> per_dev(64);
  at::Tensor& t = per_dev[dev.index() < 0 ? 0 : dev.index()];
  if (!t.defined()) t = at::zeros({4}, at::TensorOptions().dtype(at::kInt).device(dev));
  return t;
}

// Reads and clears the device status word (synchronises). Non-zero: a bounded wait inside a
// kernel ran out and the kernel returned early.
int64_t read_status(int64_t device_index) {
  at::Device dev(at::kCUDA, static_cast<c10::DeviceIndex>(device_index));
  at::Tensor& t = status_tensor(dev);
  int64_t v = t.cpu()[0].item<int>();
  if (v != 0) t.zero_();
  return v;
}

using GemmTuple = std::tuple<at::Tensor, bool, at::Tensor, bool, at::Tensor, int64_t, int64_t, int64_t, OptT, OptT,
                             OptT, OptT, OptT, int64_t, int64_t, int64_t>;

const void* opt_ptr(const OptT& t) { return (t.has_value() && t->defined()) ? t->data_ptr() : nullptr; }

void fill_call(wx::GemmCall& c, const GemmTuple& g) {
  const at::Tensor& A = std::get<0>(g);
  const at::Tensor& B = std::get<2>(g);
  const at::Tensor& D = std::get<4>(g);
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && D.is_cuda(), "gemm: CUDA tensors required");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16, "gemm: bf16 operands");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && D.dim() == 2, "gemm: 2-D tensors");
  TORCH_CHECK(A.stride(1) == 1 && B.stride(1) == 1 && D.stride(1) == 1, "gemm: unit inner stride");
  TORCH_CHECK((A.stride(0) % 8) == 0 && (B.stride(0) % 8) == 0, "gemm: operand row pitch must be a multiple of 16 B");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(A.data_ptr()) % 16) == 0 &&
                  (reinterpret_cast<uintptr_t>(B.data_ptr()) % 16) == 0,
              "gemm: operand base must be 16-byte aligned");
  c.A = A.data_ptr();
  c.lda = A.stride(0);
  c.a_mn = std::get<1>(g);
  c.a_extent_mn = c.a_mn ? A.size(1) : A.size(0);
  c.a_extent_k = c.a_mn ? A.size(0) : A.size(1);
  c.B = B.data_ptr();
  c.ldb = B.stride(0);
  c.b_mn = std::get<3>(g);
  c.b_extent_mn = c.b_mn ? B.size(1) : B.size(0);
  c.b_extent_k = c.b_mn ? B.size(0) : B.size(1);
  c.M = static_cast<int>(std::get<5>(g));
  c.N = static_cast<int>(std::get<6>(g));
  c.K = static_cast<int>(std::get<7>(g));
  c.D = D.data_ptr();
  c.ldd = D.stride(0);
  const OptT& bias = std::get<8>(g);
  const OptT& residual = std::get<9>(g);
  const OptT& row_map = std::get<10>(g);
  const OptT& dyn = std::get<11>(g);
  const OptT& D2 = std::get<12>(g);
  c.flags = static_cast<int>(std::get<13>(g));
  c.m0 = static_cast<int>(std::get<14>(g));
  c.k0 = static_cast<int>(std::get<15>(g));
  c.bias = opt_ptr(bias);
  if (c.bias) TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->is_contiguous(), "gemm: bias bf16");
  c.residual = opt_ptr(residual);
  c.ldr = c.residual ? residual->stride(0) : 0;
  if (c.residual) TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->stride(1) == 1, "gemm: residual");
  c.row_map = reinterpret_cast<const int*>(opt_ptr(row_map));
  if (c.row_map) TORCH_CHECK(row_map->scalar_type() == at::kInt, "gemm: row_map int32");
  c.dyn = reinterpret_cast<const int*>(opt_ptr(dyn));
  if (c.dyn) TORCH_CHECK(dyn->scalar_type() == at::kInt && dyn->numel() >= 4, "gemm: dyn int32[4]");
  c.D2 = const_cast<void*>(opt_ptr(D2));
  c.ldd2 = c.D2 ? D2->stride(0) : 0;
  const bool fp32 = (c.flags & wx::GEMM_OUT_FP32) != 0;
  TORCH_CHECK(D.scalar_type() == (fp32 ? at::kFloat : at::kBFloat16), "gemm: output dtype does not match flags");
  if (c.flags & wx::GEMM_ACT_SWIGLU) {
    TORCH_CHECK(!fp32 && (c.ldd % 8) == 0 && (reinterpret_cast<uintptr_t>(c.D) % 16) == 0, "gemm: swiglu output");
    if (c.D2) TORCH_CHECK((c.ldd2 % 8) == 0 && (reinterpret_cast<uintptr_t>(c.D2) % 16) == 0, "gemm: swiglu raw output");
  }
}

void gemm_grouped(const std::vector<GemmTuple>& calls, int64_t force_bn) {
  TORCH_CHECK(calls.size() >= 1 && calls.size() <= 2, "gemm: one or two problems per launch");
  wx::GemmCall cs[2];
  for (size_t i = 0; i < calls.size(); ++i) fill_call(cs[i], calls[i]);
  const at::Tensor& A0 = std::get<0>(calls[0]);
  c10::cuda::CUDAGuard guard(A0.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  int* status = status_tensor(A0.device()).data_ptr<int>();
  int rc = wx::gemm_launch(cs, static_cast<int>(calls.size()), stream, status, static_cast<int>(force_bn));
  TORCH_CHECK(rc == 0, "gemm_launch failed with code ", rc);
}

}  // namespace

void register_kernel_bindings(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm_grouped", &gemm_grouped, "tcgen05 GEMM: one or two problems in one launch");
  m.def("read_status", &read_status, "read and clear the device-side wait-timeout status");
  register_kernel_bindings(m);
}

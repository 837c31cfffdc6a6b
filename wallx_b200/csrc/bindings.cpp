// Python bindings (torch tensors -> raw-pointer launchers). This is the only translation unit
// that sees torch headers; the kernels live in plain .cu files.
//
// Reference parity: csrc/ops.cu:11-21 (the pybind table of the reference's nine ops).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdio>
#include <stdexcept>
#include <tuple>
#include <vector>

#include "attention.h"
#include "bind_common.h"
#include "comm.h"
#include "decode.h"
#include "gemm.h"
#include "kernels.h"

namespace wxb {

// Launch-failure report formatted with snprintf (no iostream on the error path).
[[noreturn]] void fail_code(const char* what, int rc) {
  char buf[160];
  snprintf(buf, sizeof(buf), "%s failed with code %d%s%s", what, rc, rc > 0 ? ": " : "",
           rc > 0 ? cudaGetErrorString(static_cast<cudaError_t>(rc)) : "");
  throw std::runtime_error(buf);
}

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
  c.d_rows = D.size(0);
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
  if (c.flags & wx::GEMM_SWIGLU_BWD) {
    TORCH_CHECK(!fp32 && c.D2 != nullptr && (c.ldd % 8) == 0 && (c.ldd2 % 8) == 0 &&
                    (reinterpret_cast<uintptr_t>(c.D) % 16) == 0 && (reinterpret_cast<uintptr_t>(c.D2) % 16) == 0 &&
                    D.size(1) >= 2 * c.N && D2->size(1) >= 2 * c.N && c.row_map == nullptr && c.bias == nullptr,
                "gemm: swiglu-backward epilogue needs bf16 [*, 2N] output and saved raw gate/up values");
  }
  if (c.flags & wx::GEMM_ACT_SWIGLU) {
    TORCH_CHECK(!fp32 && (c.ldd % 8) == 0 && (reinterpret_cast<uintptr_t>(c.D) % 16) == 0, "gemm: swiglu output");
    if (c.D2) TORCH_CHECK((c.ldd2 % 8) == 0 && (reinterpret_cast<uintptr_t>(c.D2) % 16) == 0, "gemm: swiglu raw output");
  }
}

}  // namespace wxb

namespace {

using wxb::fail_code;
using wxb::fill_call;
using wxb::GemmTuple;
using wxb::OptT;
using wxb::status_tensor;

void gemm_grouped(const std::vector<GemmTuple>& calls, int64_t force_bn) {
  TORCH_CHECK(calls.size() >= 1 && calls.size() <= 2, "gemm: one or two problems per launch");
  wx::GemmCall cs[2];
  for (size_t i = 0; i < calls.size(); ++i) fill_call(cs[i], calls[i]);
  const at::Tensor& A0 = std::get<0>(calls[0]);
  c10::cuda::CUDAGuard guard(A0.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  int* status = status_tensor(A0.device()).data_ptr<int>();
  int rc = wx::gemm_launch(cs, static_cast<int>(calls.size()), stream, status, static_cast<int>(force_bn));
  if (rc != 0) fail_code("gemm_launch", rc);
}

// One or two GEMMs whose weight operands (tuple element 2 = the local staging buffers) are gathered
// from the ranks' shards while the kernel runs. peers[i] are the raw device addresses of problem
// i's shards, one per rank.
void gemm_ag(const std::vector<GemmTuple>& calls, const std::vector<std::vector<int64_t>>& peers,
             const std::vector<at::Tensor>& flags, int64_t rank, const std::vector<int64_t>& rows_per_rank,
             int64_t n_pullers, const std::vector<int64_t>& epoch) {
  const size_t n = calls.size();
  TORCH_CHECK(n >= 1 && n <= 2 && peers.size() == n && flags.size() == n && rows_per_rank.size() == n && epoch.size() == n,
              "gemm_ag: one or two problems, one entry per problem in every list");
  wx::GemmCall cs[2];
  wx::AgInfo ags[2] = {};
  for (size_t i = 0; i < n; ++i) {
    fill_call(cs[i], calls[i]);
    TORCH_CHECK(peers[i].size() >= 1 && peers[i].size() <= 8, "gemm_ag: 1..8 ranks");
    TORCH_CHECK(flags[i].is_cuda() && flags[i].scalar_type() == at::kInt && flags[i].is_contiguous(), "gemm_ag: flags int32");
    const at::Tensor& W = std::get<2>(calls[i]);
    TORCH_CHECK(W.is_contiguous(), "gemm_ag: staging must be contiguous");
    TORCH_CHECK(W.size(0) == static_cast<int64_t>(peers[i].size()) * rows_per_rank[i],
                "gemm_ag: staging rows != world * rows_per_rank");
    TORCH_CHECK(flags[i].numel() >= (W.size(0) + 255) / 256, "gemm_ag: one flag per 256 weight rows");
    wx::AgInfo& ag = ags[i];
    for (size_t r = 0; r < peers[i].size(); ++r)
      ag.peer[r] = reinterpret_cast<const void*>(static_cast<uintptr_t>(peers[i][r]));
    ag.staging = W.data_ptr();
    ag.flags = flags[i].data_ptr<int>();
    ag.world = static_cast<int>(peers[i].size());
    ag.rank = static_cast<int>(rank);
    ag.rows_per_rank = static_cast<int>(rows_per_rank[i]);
    ag.n_pullers = static_cast<int>(n_pullers);
    ag.epoch = static_cast<int>(epoch[i]);
  }
  const at::Tensor& W0 = std::get<2>(calls[0]);
  c10::cuda::CUDAGuard guard(W0.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  int* status = status_tensor(W0.device()).data_ptr<int>();
  int rc = wx::gemm_ag_launch(cs, ags, static_cast<int>(n), stream, status);
  if (rc != 0) fail_code("gemm_ag_launch", rc);
}

bool view2d_ok(const at::Tensor& t) {
  return t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1 && (t.stride(0) % 8) == 0 &&
         (reinterpret_cast<uintptr_t>(t.data_ptr()) % 16) == 0;
}

wx::AttnShape attn_shape(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, int64_t hq, int64_t hkv,
                         int64_t d, double scale, bool has_bidir, bool causal_self) {
  TORCH_CHECK(view2d_ok(q) && view2d_ok(k) && view2d_ok(v), "attention: q/k/v must be bf16 2-D views with 16-byte aligned rows");
  TORCH_CHECK(q.size(1) == hq * d && k.size(1) == hkv * d && v.size(1) == hkv * d && k.size(0) == v.size(0),
              "attention: shape mismatch");
  wx::AttnShape s;
  s.Tq = q.size(0);
  s.Tk = k.size(0);
  s.hq = hq;
  s.hkv = hkv;
  s.D = d;
  s.ld_q = q.stride(0);
  s.ld_k = k.stride(0);
  s.ld_v = v.stride(0);
  s.scale = static_cast<float>(scale);
  s.has_bidir = has_bidir ? 1 : 0;
  s.causal_self = causal_self ? 1 : 0;
  return s;
}

std::tuple<at::Tensor, at::Tensor> attn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                            const at::Tensor& qtab, const at::Tensor& ktab, int64_t hq, int64_t hkv,
                                            int64_t d, double scale, bool has_bidir) {
  wx::AttnShape s = attn_shape(q, k, v, hq, hkv, d, scale, has_bidir, false);
  TORCH_CHECK(qtab.scalar_type() == at::kInt && qtab.is_contiguous() && qtab.size(0) == s.Tq && qtab.size(1) == 4);
  TORCH_CHECK(ktab.scalar_type() == at::kInt && ktab.is_contiguous() && ktab.size(0) == s.Tk && ktab.size(1) == 4);
  c10::cuda::CUDAGuard guard(q.device());
  at::Tensor out = at::empty({s.Tq, hq * d}, q.options());
  at::Tensor lse = at::empty({hq, s.Tq}, q.options().dtype(at::kFloat));
  int rc = wx::attn_fwd(s, q.data_ptr(), k.data_ptr(), v.data_ptr(), qtab.data_ptr(), ktab.data_ptr(), out.data_ptr(),
                        out.stride(0), lse.data_ptr<float>(), at::cuda::getCurrentCUDAStream(),
                        status_tensor(q.device()).data_ptr<int>());
  TORCH_CHECK(rc == 0, "attn_fwd failed with code ", rc);
  return {out, lse};
}

// dq / dk / dv are written in place into caller-provided (possibly strided) views.
void attn_bwd(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
              const at::Tensor& out, const at::Tensor& lse, const at::Tensor& qtab, const at::Tensor& ktab,
              at::Tensor& dq, at::Tensor& dk, at::Tensor& dv, int64_t hq, int64_t hkv, int64_t d, double scale,
              bool has_bidir, bool causal_self) {
  wx::AttnShape s = attn_shape(q, k, v, hq, hkv, d, scale, has_bidir, causal_self);
  TORCH_CHECK(view2d_ok(dout) && view2d_ok(out) && view2d_ok(dq) && view2d_ok(dk) && view2d_ok(dv), "attn_bwd: views");
  c10::cuda::CUDAGuard guard(q.device());
  auto fo = q.options().dtype(at::kFloat);
  at::Tensor delta = at::empty({hq, s.Tq}, fo);
  const int rep = hq / hkv;
  at::Tensor pk, pv;
  float *ppk = nullptr, *ppv = nullptr;
  if (rep > 1) {
    pk = at::empty({rep, s.Tk, hkv * d}, fo);
    pv = at::empty({rep, s.Tk, hkv * d}, fo);
    ppk = pk.data_ptr<float>();
    ppv = pv.data_ptr<float>();
  }
  int rc = wx::attn_bwd(s, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), out.stride(0), dout.data_ptr(),
                        dout.stride(0), lse.data_ptr<float>(), qtab.data_ptr(), ktab.data_ptr(), delta.data_ptr<float>(),
                        dq.data_ptr(), dq.stride(0), dk.data_ptr(), dk.stride(0), dv.data_ptr(), dv.stride(0), ppk, ppv,
                        at::cuda::getCurrentCUDAStream(), status_tensor(q.device()).data_ptr<int>());
  TORCH_CHECK(rc == 0, "attn_bwd failed with code ", rc);
}

}  // namespace

void register_kernel_bindings(pybind11::module_& m);
void register_block_bindings(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm_ag", &gemm_ag, "GEMM with the weight all-gather fused in (peer loads over NVLink)");
  m.def("gemm_grouped", &gemm_grouped, "tcgen05 GEMM: one or two problems in one launch");
  m.def("checked_build", []() { return wx::gemm_checked_build() != 0; }, "true when the kernels were compiled with -DWX_CHECK");
  m.def("check_report", [](bool clear) {
    // one record per translation unit: {unit: [first violating site, violations, value, value]} (synchronises)
    cudaDeviceSynchronize();
    pybind11::dict out;
    long long r[4];
    struct Unit { const char* name; int (*read)(long long*, int); };
    const Unit units[] = {{"gemm", &wx::gemm_check_read}, {"attention", &wx::attn_check_read}, {"kernels", &wx::kernels_check_read},
                          {"index", &wx::index_check_read}, {"comm", &wx::comm_check_read},
                          {"decode", &wx::decode_check_read}};
    for (const Unit& u : units) {
      const int rc = u.read(r, clear ? 1 : 0);
      if (rc != 0) wxb::fail_code("check_report", rc);
      out[u.name] = std::vector<long long>{r[0], r[1], r[2], r[3]};
    }
    return out;
  }, pybind11::arg("clear") = true, "range-check records of the debug build (all zeros in a release build)");
  m.def("gemm_tile_rates", [](const std::vector<double>& set) {
    if (set.size() == 4) wx::gemm_set_tile_rates(set.data());
    std::vector<double> cur(4);
    wx::gemm_get_tile_rates(cur.data());
    return cur;
  }, pybind11::arg("set") = std::vector<double>(), "get (and with four values: set) the per-tile-shape rates of the tile cost model");
  m.def("read_status", &wxb::read_status, "read and clear the device-side wait-timeout status");
  m.def("status_tensor", [](int64_t device_index) {
    return wxb::status_tensor(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device_index)));
  }, "the device-side status words themselves (int32[4]; word 0 non-zero after a wait ran out)");
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
  register_kernel_bindings(m);
  register_block_bindings(m);
}

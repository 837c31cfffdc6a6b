// Bindings of the non-GEMM kernels (allocation and checks here, arithmetic in kernels.cu).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "comm.h"
#include "decode.h"
#include "launch.h"
#include "kernels.h"

namespace {

using OptT = c10::optional<at::Tensor>;

#define WX_CHECK_RC(rc, what) TORCH_CHECK((rc) == 0, what, " failed with code ", (rc))

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream(); }

void check_bf16(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), name, ": contiguous CUDA bf16 expected");
}
const int* opt_int(const OptT& t) {
  if (!t.has_value() || !t->defined() || t->numel() == 0) return nullptr;
  TORCH_CHECK(t->scalar_type() == at::kInt && t->is_cuda() && t->is_contiguous(), "int32 CUDA tensor expected");
  return t->data_ptr<int>();
}

// `zero_pad`: with a row map, rows of the output that no token maps to are zero-filled. The backward
// pass reduces over padded segments and needs that; inference may skip it (those rows only feed
// accumulator rows that are never stored).
std::tuple<at::Tensor, at::Tensor> rms_norm_fwd(const at::Tensor& x, const at::Tensor& w, double eps, const OptT& dest,
                                                int64_t out_rows, bool zero_pad) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  c10::cuda::CUDAGuard g(x.device());
  const int T = x.size(0), C = x.size(1);
  const int* dp = opt_int(dest);
  at::Tensor y = dp ? (zero_pad ? at::zeros({out_rows, C}, x.options()) : at::empty({out_rows, C}, x.options()))
                    : at::empty({T, C}, x.options());
  at::Tensor rstd = at::empty({T}, x.options().dtype(at::kFloat));
  WX_CHECK_RC(wx::rms_norm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), dp, T, C,
                               static_cast<float>(eps), cur_stream()),
              "rms_norm_fwd");
  return {y, rstd};
}

std::tuple<at::Tensor, at::Tensor> rms_norm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w,
                                                const at::Tensor& rstd, const OptT& dest) {
  check_bf16(dy, "dy");
  check_bf16(x, "x");
  c10::cuda::CUDAGuard g(x.device());
  const int T = x.size(0), C = x.size(1);
  at::Tensor dx = at::empty_like(x);
  at::Tensor dw = at::empty_like(w);
  at::Tensor partial = at::empty({wx::rms_norm_bwd_blocks(T), C}, x.options().dtype(at::kFloat));
  WX_CHECK_RC(wx::rms_norm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), opt_int(dest),
                               dx.data_ptr(), partial.data_ptr<float>(), dw.data_ptr(), T, C, cur_stream()),
              "rms_norm_bwd");
  return {dx, dw};
}

at::Tensor swiglu_bwd(const at::Tensor& dh, const at::Tensor& gu) {
  TORCH_CHECK(dh.is_cuda() && gu.is_cuda() && dh.scalar_type() == at::kBFloat16 && gu.scalar_type() == at::kBFloat16);
  TORCH_CHECK(dh.dim() == 2 && gu.dim() == 2 && dh.stride(1) == 1 && gu.stride(1) == 1 && gu.size(1) == 2 * dh.size(1));
  c10::cuda::CUDAGuard g(gu.device());
  at::Tensor dgu = at::empty({gu.size(0), gu.size(1)}, gu.options());
  WX_CHECK_RC(wx::swiglu_bwd(dh.data_ptr(), gu.data_ptr(), dgu.data_ptr(), gu.size(0), gu.size(1), dh.stride(0),
                             gu.stride(0), cur_stream()),
              "swiglu_bwd");
  return dgu;
}

at::Tensor rope_qk(const at::Tensor& qkv, const at::Tensor& cos_t, const at::Tensor& sin_t, int64_t n_rot, int64_t D,
                   bool inverse) {
  check_bf16(qkv, "qkv");
  TORCH_CHECK(cos_t.scalar_type() == at::kFloat && sin_t.scalar_type() == at::kFloat && cos_t.is_contiguous() &&
              sin_t.is_contiguous() && cos_t.size(0) == qkv.size(0) && cos_t.size(1) == D,
              "rope_qk: cos/sin must be fp32 [T, D]");
  c10::cuda::CUDAGuard g(qkv.device());
  at::Tensor out = at::empty_like(qkv);
  WX_CHECK_RC(wx::rope_qk(qkv.data_ptr(), out.data_ptr(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), qkv.size(0),
                          qkv.size(1), n_rot, D, inverse ? 1 : 0, cur_stream()),
              "rope_qk");
  return out;
}

// Rotary on q and k of a packed q|k|v buffer (q in place); rotated k and v go to the rows' slots of the cache.
void rope_cache(at::Tensor& qkv, const at::Tensor& cos_t, const at::Tensor& sin_t, const at::Tensor& cache_rows,
                at::Tensor& cache, int64_t hq, int64_t hkv, int64_t D) {
  check_bf16(qkv, "qkv");
  TORCH_CHECK(qkv.is_contiguous() && cache.is_cuda() && cache.scalar_type() == at::kBFloat16 && cache.dim() == 2 &&
              cache.stride(1) == 1, "rope_cache: contiguous bf16 qkv and a bf16 [rows, >= 2 hkv D] cache");
  TORCH_CHECK(cos_t.scalar_type() == at::kFloat && sin_t.scalar_type() == at::kFloat && cos_t.is_contiguous() &&
              sin_t.is_contiguous() && cos_t.size(0) == qkv.size(0) && cos_t.size(1) == D && sin_t.size(0) == qkv.size(0),
              "rope_cache: cos/sin must be fp32 [T, D]");
  TORCH_CHECK(cache_rows.is_cuda() && cache_rows.scalar_type() == at::kLong && cache_rows.is_contiguous() &&
              cache_rows.numel() == qkv.size(0), "rope_cache: int64 cache row per token");
  c10::cuda::CUDAGuard g(qkv.device());
  WX_CHECK_RC(wx::rope_cache(qkv.data_ptr(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), cache_rows.data_ptr<int64_t>(),
                             cache.data_ptr(), qkv.size(0), qkv.size(1), hq, hkv, D, cache.stride(0), cache.size(0),
                             cur_stream()),
              "rope_cache");
}

bool attn_decode_supported(int64_t Tq, int64_t hq, int64_t hkv, int64_t D) {
  return wx::attn_decode_supported(static_cast<int>(Tq), static_cast<int>(hq), static_cast<int>(hkv), static_cast<int>(D));
}

// Few query rows over cached keys / values (row-strided views are fine); tables as for the tensor-core kernel.
at::Tensor attn_decode(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& qtab,
                       const at::Tensor& ktab, int64_t hq, int64_t hkv, int64_t D, double scale, int64_t max_keys) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
              v.scalar_type() == at::kBFloat16 && q.dim() == 2 && k.dim() == 2 && v.dim() == 2 && q.stride(1) == 1 &&
              k.stride(1) == 1 && v.stride(1) == 1, "attn_decode: bf16 row-strided q, k, v");
  TORCH_CHECK(q.size(1) == hq * D && k.size(1) == hkv * D && v.size(1) == hkv * D && k.size(0) == v.size(0));
  TORCH_CHECK(qtab.scalar_type() == at::kInt && qtab.is_contiguous() && qtab.size(0) == q.size(0) && qtab.size(1) == 4);
  TORCH_CHECK(ktab.scalar_type() == at::kInt && ktab.is_contiguous() && ktab.size(0) == k.size(0) && ktab.size(1) == 4);
  TORCH_CHECK((reinterpret_cast<uintptr_t>(q.data_ptr()) % 16) == 0 && (reinterpret_cast<uintptr_t>(k.data_ptr()) % 16) == 0 &&
              (reinterpret_cast<uintptr_t>(v.data_ptr()) % 16) == 0, "attn_decode: 16-byte aligned operands");
  c10::cuda::CUDAGuard g(q.device());
  at::Tensor out = at::empty({q.size(0), hq * D}, q.options());
  WX_CHECK_RC(wx::attn_decode(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), qtab.data_ptr(),
                              ktab.data_ptr(), out.data_ptr(), out.stride(0), q.size(0), k.size(0), hq, hkv, D,
                              static_cast<float>(scale), static_cast<int>(max_keys), cur_stream()),
              "attn_decode");
  return out;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> route_plan(const at::Tensor& types, int64_t E, int64_t rows) {
  TORCH_CHECK(types.is_cuda() && types.scalar_type() == at::kInt && types.is_contiguous(), "route_plan: int32 types");
  c10::cuda::CUDAGuard g(types.device());
  const int T = types.numel();
  auto io = types.options();
  at::Tensor dest = at::empty({T}, io), seg = at::empty({E, 4}, io), segk = at::empty({E, 4}, io),
             inv = at::empty({rows}, io);
  WX_CHECK_RC(wx::route_plan(types.data_ptr<int>(), T, E, rows, dest.data_ptr<int>(), seg.data_ptr<int>(),
                             segk.data_ptr<int>(), inv.data_ptr<int>(), cur_stream()),
              "route_plan");
  return {dest, seg, segk, inv};
}

at::Tensor permute_rows(const at::Tensor& x, const at::Tensor& dest, int64_t rows) {
  check_bf16(x, "x");
  c10::cuda::CUDAGuard g(x.device());
  at::Tensor out = at::zeros({rows, x.size(1)}, x.options());
  WX_CHECK_RC(wx::permute_rows(x.data_ptr(), dest.data_ptr<int>(), out.data_ptr(), x.size(0), x.size(1), cur_stream(),
                               static_cast<int>(rows)),
              "permute_rows");
  return out;
}

at::Tensor gather_rows(const at::Tensor& x, const at::Tensor& idx) {
  check_bf16(x, "x");
  TORCH_CHECK(idx.scalar_type() == at::kInt && idx.is_cuda() && idx.is_contiguous());
  c10::cuda::CUDAGuard g(x.device());
  at::Tensor out = at::empty({idx.numel(), x.size(1)}, x.options());
  WX_CHECK_RC(wx::gather_rows(x.data_ptr(), idx.data_ptr<int>(), out.data_ptr(), idx.numel(), x.size(1), cur_stream(),
                              static_cast<int>(x.size(0))),
              "gather_rows");
  return out;
}

at::Tensor column_sum(const at::Tensor& x) {
  check_bf16(x, "x");
  c10::cuda::CUDAGuard g(x.device());
  at::Tensor acc = at::empty({wx::column_sum_slabs(x.size(0)), x.size(1)}, x.options().dtype(at::kFloat));
  at::Tensor out = at::empty({x.size(1)}, x.options());
  WX_CHECK_RC(wx::column_sum(x.data_ptr(), acc.data_ptr<float>(), out.data_ptr(), x.size(0), x.size(1), cur_stream()),
              "column_sum");
  return out;
}

void ce_fwd(const at::Tensor& logits, const at::Tensor& labels, at::Tensor& loss, at::Tensor& lse, at::Tensor& pred) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.stride(1) == 1);
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous() && pred.scalar_type() == at::kLong);
  c10::cuda::CUDAGuard g(logits.device());
  WX_CHECK_RC(wx::ce_fwd(logits.data_ptr(), reinterpret_cast<const long*>(labels.data_ptr<int64_t>()),
                         loss.data_ptr<float>(), lse.data_ptr<float>(), reinterpret_cast<long*>(pred.data_ptr<int64_t>()),
                         logits.size(0), logits.size(1), logits.stride(0), cur_stream()),
              "ce_fwd");
}

void ce_bwd(at::Tensor& logits, const at::Tensor& labels, const at::Tensor& lse, const at::Tensor& dloss) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.stride(1) == 1);
  c10::cuda::CUDAGuard g(logits.device());
  WX_CHECK_RC(wx::ce_bwd(logits.data_ptr(), reinterpret_cast<const long*>(labels.data_ptr<int64_t>()),
                         lse.data_ptr<float>(), dloss.data_ptr<float>(), logits.size(0), logits.size(1),
                         logits.stride(0), cur_stream()),
              "ce_bwd");
}

void sumsq_bf16(const at::Tensor& g, at::Tensor& out) {
  TORCH_CHECK(g.is_cuda() && g.scalar_type() == at::kBFloat16 && g.is_contiguous() && out.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(g.device());
  WX_CHECK_RC(wx::sumsq_bf16(g.data_ptr(), g.numel(), out.data_ptr<float>(), cur_stream()), "sumsq_bf16");
}

void adamw_step(at::Tensor& p16, at::Tensor& p32, at::Tensor& m, at::Tensor& v, const at::Tensor& g,
                const at::Tensor& hyper, const OptT& norm_sq) {
  TORCH_CHECK(p16.is_cuda() && p16.scalar_type() == at::kBFloat16 && g.scalar_type() == at::kBFloat16);
  TORCH_CHECK(p32.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat);
  TORCH_CHECK(p16.is_contiguous() && p32.is_contiguous() && m.is_contiguous() && v.is_contiguous() && g.is_contiguous());
  const int64_t n = p16.numel();
  TORCH_CHECK(p32.numel() == n && m.numel() == n && v.numel() == n && g.numel() == n, "adamw: size mismatch");
  TORCH_CHECK(hyper.scalar_type() == at::kFloat && hyper.numel() >= 9 && hyper.is_cuda());
  c10::cuda::CUDAGuard guard(p16.device());
  const float* ns = (norm_sq.has_value() && norm_sq->defined()) ? norm_sq->data_ptr<float>() : nullptr;
  WX_CHECK_RC(wx::adamw_step(p16.data_ptr(), p32.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                             g.data_ptr(), n, hyper.data_ptr<float>(), ns, cur_stream()),
              "adamw_step");
}

wx::PeerPtrs peer_ptrs(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() >= 1 && ptrs.size() <= wx::kMaxPeers, "1..8 peers");
  wx::PeerPtrs pp{};
  for (size_t i = 0; i < ptrs.size(); ++i) pp.p[i] = reinterpret_cast<void*>(ptrs[i]);
  return pp;
}

void symm_barrier(const std::vector<int64_t>& flag_ptrs, int64_t rank, int64_t epoch, at::Tensor& status,
                  int64_t timeout_ms) {
  WX_CHECK_RC(wx::symm_barrier(peer_ptrs(flag_ptrs), rank, flag_ptrs.size(), epoch, status.data_ptr<int>(), cur_stream(),
                               static_cast<long>(timeout_ms)),
              "symm_barrier");
}

void rs_reduce(const std::vector<int64_t>& grad_ptrs, const at::Tensor& table, at::Tensor& out, at::Tensor& sumsq) {
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.dim() == 2 && table.size(1) == 3 && table.is_contiguous());
  TORCH_CHECK(out.scalar_type() == at::kFloat && sumsq.scalar_type() == at::kFloat);
  WX_CHECK_RC(wx::rs_reduce(peer_ptrs(grad_ptrs), reinterpret_cast<const wx::ShardDesc*>(table.data_ptr<int64_t>()),
                            table.size(0), grad_ptrs.size(), out.data_ptr<float>(), sumsq.data_ptr<float>(), cur_stream()),
              "rs_reduce");
}

void ag_push(const std::vector<int64_t>& param_ptrs, const at::Tensor& table, int64_t rank) {
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.size(1) == 3 && table.is_contiguous());
  WX_CHECK_RC(wx::ag_push(peer_ptrs(param_ptrs), reinterpret_cast<const wx::ShardDesc*>(table.data_ptr<int64_t>()),
                          table.size(0), rank, param_ptrs.size(), cur_stream()),
              "ag_push");
}

void ag_push_multicast(int64_t mc_ptr, int64_t local_ptr, const at::Tensor& table) {
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.size(1) == 3 && table.is_contiguous());
  TORCH_CHECK(mc_ptr != 0 && local_ptr != 0, "ag_push_multicast: no multicast mapping");
  WX_CHECK_RC(wx::ag_push_multicast(reinterpret_cast<void*>(mc_ptr), reinterpret_cast<const void*>(local_ptr),
                                    reinterpret_cast<const wx::ShardDesc*>(table.data_ptr<int64_t>()), table.size(0), cur_stream()),
              "ag_push_multicast");
}

void small_allreduce_write(const std::vector<int64_t>& scratch_ptrs, const at::Tensor& vals, int64_t rank) {
  TORCH_CHECK(vals.is_cuda() && vals.scalar_type() == at::kFloat && vals.is_contiguous());
  WX_CHECK_RC(wx::small_allreduce_write(peer_ptrs(scratch_ptrs), vals.data_ptr<float>(), vals.numel(), rank,
                                        scratch_ptrs.size(), cur_stream()),
              "small_allreduce_write");
}

void small_allreduce_sum(const at::Tensor& my_scratch, at::Tensor& out, int64_t world) {
  WX_CHECK_RC(wx::small_allreduce_sum(my_scratch.data_ptr<float>(), out.data_ptr<float>(), out.numel(), world, cur_stream()),
              "small_allreduce_sum");
}

void adamw_step_f32g(at::Tensor& p16, at::Tensor& p32, at::Tensor& m, at::Tensor& v, const at::Tensor& g,
                     const at::Tensor& hyper, const OptT& norm_sq) {
  TORCH_CHECK(p16.scalar_type() == at::kBFloat16 && g.scalar_type() == at::kFloat && p32.scalar_type() == at::kFloat);
  TORCH_CHECK(p16.is_contiguous() && p32.is_contiguous() && m.is_contiguous() && v.is_contiguous() && g.is_contiguous());
  const int64_t n = p16.numel();
  TORCH_CHECK(p32.numel() == n && m.numel() == n && v.numel() == n && g.numel() == n, "adamw: size mismatch");
  c10::cuda::CUDAGuard guard(p16.device());
  const float* ns = (norm_sq.has_value() && norm_sq->defined()) ? norm_sq->data_ptr<float>() : nullptr;
  WX_CHECK_RC(wx::adamw_step_f32g(p16.data_ptr(), p32.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                                  g.data_ptr<float>(), n, hyper.data_ptr<float>(), ns, cur_stream()),
              "adamw_step_f32g");
}

std::tuple<at::Tensor, at::Tensor> rope_index(const at::Tensor& ids, const OptT& mask, const at::Tensor& img_grid,
                                              const at::Tensor& vid_grid, const at::Tensor& sec_per_grid, int64_t merge,
                                              int64_t image_id, int64_t video_id, int64_t vstart_id, double tps) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.dim() == 2 && ids.is_contiguous(), "rope_index: ids");
  TORCH_CHECK(img_grid.scalar_type() == at::kInt && vid_grid.scalar_type() == at::kInt && img_grid.is_contiguous() &&
              vid_grid.is_contiguous() && sec_per_grid.scalar_type() == at::kFloat, "rope_index: grids");
  c10::cuda::CUDAGuard g(ids.device());
  const int B = ids.size(0), S = ids.size(1);
  at::Tensor pos = at::empty({3, B, S}, ids.options());
  at::Tensor deltas = at::empty({B, 1}, ids.options());
  at::Tensor status = at::zeros({1}, ids.options().dtype(at::kInt));
  WX_CHECK_RC(wx::rope_index(reinterpret_cast<const long*>(ids.data_ptr<int64_t>()), opt_int(mask), img_grid.data_ptr<int>(),
                             img_grid.size(0), vid_grid.data_ptr<int>(), vid_grid.size(0),
                             sec_per_grid.numel() ? sec_per_grid.data_ptr<float>() : nullptr, B, S, merge, image_id,
                             video_id, vstart_id, static_cast<float>(tps), reinterpret_cast<long*>(pos.data_ptr<int64_t>()),
                             reinterpret_cast<long*>(deltas.data_ptr<int64_t>()), status.data_ptr<int>(), cur_stream()),
              "rope_index");
  return {pos, deltas};
}

at::Tensor vit_rot_pos(const at::Tensor& inv_freq, const at::Tensor& grid, int64_t merge, int64_t total) {
  TORCH_CHECK(inv_freq.is_cuda() && inv_freq.scalar_type() == at::kFloat && grid.is_cuda() && grid.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard g(grid.device());
  const int F = inv_freq.numel();
  at::Tensor out = at::empty({total, 2 * F}, inv_freq.options());
  WX_CHECK_RC(wx::vit_rot_pos(inv_freq.data_ptr<float>(), F, grid.data_ptr<int>(), grid.size(0), merge,
                              out.data_ptr<float>(), total, cur_stream()),
              "vit_rot_pos");
  return out;
}

std::tuple<at::Tensor, at::Tensor> vit_window_index(const at::Tensor& grid, int64_t vw, int64_t merge, int64_t n_merged,
                                                    int64_t n_windows) {
  TORCH_CHECK(grid.is_cuda() && grid.scalar_type() == at::kInt && grid.is_contiguous());
  c10::cuda::CUDAGuard g(grid.device());
  at::Tensor idx = at::empty({n_merged}, grid.options().dtype(at::kLong));
  at::Tensor cu = at::empty({n_windows + 1}, grid.options());
  WX_CHECK_RC(wx::vit_window_index(grid.data_ptr<int>(), grid.size(0), vw, merge, reinterpret_cast<long*>(idx.data_ptr<int64_t>()),
                                   cu.data_ptr<int>(), cur_stream()),
              "vit_window_index");
  return {idx, cu};
}

}  // namespace

void register_kernel_bindings(pybind11::module_& m) {
  m.def("rms_norm_fwd", &rms_norm_fwd, pybind11::arg("x"), pybind11::arg("w"), pybind11::arg("eps"),
        pybind11::arg("dest"), pybind11::arg("out_rows"), pybind11::arg("zero_pad") = true);
  m.def("rms_norm_bwd", &rms_norm_bwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("rope_qk", &rope_qk);
  m.def("set_pdl", [](bool on) { wx::pdl_set(on); });
  m.def("pdl_enabled", []() { return wx::pdl_enabled(); });
  m.def("rope_cache", &rope_cache);
  m.def("attn_decode", &attn_decode);
  m.def("attn_decode_supported", &attn_decode_supported);
  m.def("route_plan", &route_plan);
  m.def("permute_rows", &permute_rows);
  m.def("gather_rows", &gather_rows);
  m.def("column_sum", &column_sum);
  m.def("ce_fwd", &ce_fwd);
  m.def("ce_bwd", &ce_bwd);
  m.def("sumsq_bf16", &sumsq_bf16);
  m.def("adamw_step", &adamw_step);
  m.def("adamw_step_f32g", &adamw_step_f32g);
  m.def("rope_index", &rope_index);
  m.def("vit_rot_pos", &vit_rot_pos);
  m.def("vit_window_index", &vit_window_index);
  m.def("symm_barrier", &symm_barrier, pybind11::arg("flag_ptrs"), pybind11::arg("rank"), pybind11::arg("epoch"),
        pybind11::arg("status"), pybind11::arg("timeout_ms") = 2000);
  m.def("rs_reduce", &rs_reduce);
  m.def("ag_push", &ag_push);
  m.def("ag_push_multicast", &ag_push_multicast);
  m.def("small_allreduce_write", &small_allreduce_write);
  m.def("small_allreduce_sum", &small_allreduce_sum);
}

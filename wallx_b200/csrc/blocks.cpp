// Whole transformer blocks as single host entry points.
//
// One call enqueues every kernel of a pre-norm attention + FFN block (forward or backward): RMSNorm, fused QKV GEMM,
// rotary, varlen attention, output projection with the residual add in its epilogue, RMSNorm (with the token-type
// permutation fused in for the dual-expert FFN), gate/up GEMM with the SwiGLU epilogue, down GEMM with un-permute and
// residual in its epilogue -- and the matching dgrad / wgrad / reduction kernels in backward. The kernels are the
// same ones the operator-by-operator Python path launches, in the same order with the same arguments, so results are
// bit-identical; what goes away is the host time between launches (Python modules, autograd nodes, argument
// conversion: more than 100 us per kernel), which otherwise bounds the training step.
//
// Serves the decoder layer (dual-expert or dense FFN, no biases except q/k/v;
// reference: Qwen2_5_VLDecoderLayer_with_MoE, modeling_qwen2_5_vl_act.py:172-273) and the vision block (biased
// projections and SwiGLU MLP; reference: Qwen2_5_VLVisionBlock, modeling_qwen2_5_vl.py:365-391).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <tuple>
#include <vector>

#include "attention.h"
#include "bind_common.h"
#include "gemm.h"
#include "kernels.h"

namespace {

using at::Tensor;
using wxb::OptT;

std::atomic<long> g_launches{0};

// A GEMM weight operand as Python hands it over:
// (w, gradient sink or None, peer shard addresses (empty: resident), ready flags or None, rows per rank, rank,
//  copy CTAs, epoch of this call). For a row-sharded weight `w` is its staging view.
using WTuple = std::tuple<Tensor, OptT, std::vector<int64_t>, OptT, int64_t, int64_t, int64_t, int64_t>;

const Tensor& w_of(const WTuple& t) { return std::get<0>(t); }
bool has_sink(const WTuple& t) { return std::get<1>(t).has_value() && std::get<1>(t)->defined(); }
bool gathered(const WTuple& t) { return !std::get<2>(t).empty(); }

cudaStream_t cur() { return at::cuda::getCurrentCUDAStream(); }

#define WX_RC(rc, what)                                   \
  do {                                                    \
    const int rc__ = (rc);                                \
    if (rc__ != 0) wxb::fail_code(what, rc__);            \
    g_launches.fetch_add(1, std::memory_order_relaxed);   \
  } while (0)

struct Spec {
  Tensor a;
  bool a_mn = false;
  Tensor b;
  bool b_mn = false;
  Tensor out;
  int64_t M = -1, N = -1, K = -1;
  OptT bias, residual, row_map, dyn, out2;
  int64_t flags = 0;
};

wxb::GemmTuple to_tuple(const Spec& s) {
  const int64_t M = s.M >= 0 ? s.M : (s.a_mn ? s.a.size(1) : s.a.size(0));
  const int64_t N = s.N >= 0 ? s.N : (s.b_mn ? s.b.size(1) : s.b.size(0));
  const int64_t K = s.K >= 0 ? s.K : (s.a_mn ? s.a.size(0) : s.a.size(1));
  return wxb::GemmTuple(s.a, s.a_mn, s.b, s.b_mn, s.out, M, N, K, s.bias, s.residual, s.row_map, s.dyn, s.out2, s.flags,
                        0, 0);
}

void launch_plain(const Spec* specs, int n, int* status) {
  wx::GemmCall cs[2];
  for (int i = 0; i < n; ++i) wxb::fill_call(cs[i], to_tuple(specs[i]));
  WX_RC(wx::gemm_launch(cs, n, cur(), status, 0), "gemm_launch");
}

void launch_gathered(const Spec* specs, const WTuple* const* ws, int n, int* status) {
  wx::GemmCall cs[2];
  wx::AgInfo ags[2] = {};
  for (int i = 0; i < n; ++i) {
    wxb::fill_call(cs[i], to_tuple(specs[i]));
    const WTuple& w = *ws[i];
    const auto& peers = std::get<2>(w);
    const Tensor& flags = *std::get<3>(w);
    TORCH_CHECK(peers.size() >= 1 && peers.size() <= 8, "block: 1..8 ranks");
    TORCH_CHECK(specs[i].b.is_contiguous(), "block: staging must be contiguous");
    for (size_t r = 0; r < peers.size(); ++r) ags[i].peer[r] = reinterpret_cast<const void*>(static_cast<uintptr_t>(peers[r]));
    ags[i].staging = specs[i].b.data_ptr();
    ags[i].flags = flags.data_ptr<int>();
    ags[i].world = static_cast<int>(peers.size());
    ags[i].rank = static_cast<int>(std::get<5>(w));
    ags[i].rows_per_rank = static_cast<int>(std::get<4>(w));
    ags[i].n_pullers = static_cast<int>(std::get<6>(w));
    ags[i].epoch = static_cast<int>(std::get<7>(w));
  }
  WX_RC(wx::gemm_ag_launch(cs, ags, n, cur(), status), "gemm_ag_launch");
}

// One or two problems whose B operands are the weights `ws` (nullptr entries: B is an activation).
// Resident weights take the plain GEMM; row-sharded ones are gathered from their owners inside the launch.
void launch(std::vector<Spec>& specs, std::vector<const WTuple*> ws, int* status) {
  const int n = static_cast<int>(specs.size());
  TORCH_CHECK(n >= 1 && n <= 2 && static_cast<int>(ws.size()) == n);
  bool any = false, all = true;
  for (int i = 0; i < n; ++i) {
    const bool g = ws[i] != nullptr && gathered(*ws[i]);
    any |= g;
    all &= g;
  }
  if (!any) return launch_plain(specs.data(), n, status);
  if (all && (n == 1 || specs[0].b.data_ptr() != specs[1].b.data_ptr())) return launch_gathered(specs.data(), ws.data(), n, status);
  for (int i = 0; i < n; ++i) {
    if (ws[i] != nullptr && gathered(*ws[i])) launch_gathered(&specs[i], &ws[i], 1, status);
    else launch_plain(&specs[i], 1, status);
  }
}

// One or two problems with operands in place, while the launch's copy CTAs gather the weights `pf` (one or two
// row-sharded weights, into their staging views) for the launches that follow.
void launch_prefetching(std::vector<Spec>& specs, const std::vector<const WTuple*>& pf, int* status) {
  const int n = static_cast<int>(specs.size()), m = static_cast<int>(pf.size());
  TORCH_CHECK(n >= 1 && n <= 2 && m >= 1 && m <= 2);
  wx::GemmCall cs[2];
  for (int i = 0; i < n; ++i) wxb::fill_call(cs[i], to_tuple(specs[i]));
  wx::AgInfo ags[2] = {};
  long cols[2] = {0, 0};
  for (int i = 0; i < m; ++i) {
    const WTuple& w = *pf[i];
    const auto& peers = std::get<2>(w);
    TORCH_CHECK(peers.size() >= 1 && peers.size() <= 8 && w_of(w).is_contiguous(), "block: bad gather record");
    for (size_t r = 0; r < peers.size(); ++r) ags[i].peer[r] = reinterpret_cast<const void*>(static_cast<uintptr_t>(peers[r]));
    ags[i].staging = w_of(w).data_ptr();
    ags[i].flags = std::get<3>(w)->data_ptr<int>();
    ags[i].world = static_cast<int>(peers.size());
    ags[i].rank = static_cast<int>(std::get<5>(w));
    ags[i].rows_per_rank = static_cast<int>(std::get<4>(w));
    ags[i].n_pullers = static_cast<int>(std::get<6>(w));
    ags[i].epoch = static_cast<int>(std::get<7>(w));
    cols[i] = w_of(w).size(1);
  }
  WX_RC(wx::gemm_launch_prefetch(cs, n, ags, cols, m, cur(), status), "gemm_launch_prefetch");
}

// Backward of a block with row-sharded weights: only the first dgrad GEMM gathers its weight on the critical path; each
// weight-gradient GEMM (which needs no weight) carries the gather of the weights the following dgrad GEMMs multiply by.
bool prefetch_enabled() {
  static const bool on = [] {
    const char* e = getenv("WX_AG_PREFETCH");
    return e == nullptr || atoi(e) != 0;
  }();
  return on;
}

Tensor empty_bf16(int64_t r, int64_t c, const Tensor& like) { return at::empty({r, c}, like.options().dtype(at::kBFloat16)); }

std::pair<Tensor, Tensor> norm_fwd(const Tensor& x, const Tensor& w, double eps, const OptT& dest, int64_t rows, bool zero_pad) {
  const int T = x.size(0), C = x.size(1);
  const bool mapped = dest.has_value() && dest->defined();
  Tensor y = mapped ? (zero_pad ? at::zeros({rows, C}, x.options()) : at::empty({rows, C}, x.options())) : at::empty({T, C}, x.options());
  Tensor rstd = at::empty({T}, x.options().dtype(at::kFloat));
  WX_RC(wx::rms_norm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), mapped ? dest->data_ptr<int>() : nullptr,
                         T, C, static_cast<float>(eps), cur()),
        "rms_norm_fwd");
  return {y, rstd};
}

// dx = rms_norm backward + `add` (the gradient arriving over the residual path, added inside the kernel), dw
std::pair<Tensor, Tensor> norm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, const OptT& dest,
                                   const Tensor& add) {
  const int T = x.size(0), C = x.size(1);
  const bool mapped = dest.has_value() && dest->defined();
  Tensor dx = at::empty_like(x);
  Tensor dw = at::empty_like(w);
  Tensor partial = at::empty({wx::rms_norm_bwd_blocks(T), C}, x.options().dtype(at::kFloat));
  WX_RC(wx::rms_norm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), mapped ? dest->data_ptr<int>() : nullptr,
                         dx.data_ptr(), partial.data_ptr<float>(), dw.data_ptr(), T, C, cur(), add.data_ptr()),
        "rms_norm_bwd");
  g_launches.fetch_add(1, std::memory_order_relaxed);  // the kernel plus its ordered partial reduction
  return {dx, dw};
}

Tensor col_sum(const Tensor& x) {
  Tensor acc = at::empty({wx::column_sum_slabs(x.size(0)), x.size(1)}, x.options().dtype(at::kFloat));
  Tensor out = at::empty({x.size(1)}, x.options());
  WX_RC(wx::column_sum(x.data_ptr(), acc.data_ptr<float>(), out.data_ptr(), x.size(0), x.size(1), cur()), "column_sum");
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return out;
}

// Rotates q and k in place (the block owns the buffer; the v columns stay where they are).
void rope_inplace(Tensor& t, const Tensor& cos_t, const Tensor& sin_t, int64_t n_rot, int64_t d, bool inverse) {
  WX_RC(wx::rope_qk(t.data_ptr(), t.data_ptr(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), t.size(0), t.size(1), n_rot, d,
                    inverse ? 1 : 0, cur()),
        "rope_qk");
}

wx::AttnShape attn_shape(const Tensor& qkv, int64_t hq, int64_t hkv, int64_t d, double scale, bool has_bidir, bool causal_self) {
  wx::AttnShape s;
  s.Tq = s.Tk = qkv.size(0);
  s.hq = hq;
  s.hkv = hkv;
  s.D = d;
  s.ld_q = s.ld_k = s.ld_v = qkv.stride(0);
  s.scale = static_cast<float>(scale);
  s.has_bidir = has_bidir ? 1 : 0;
  s.causal_self = causal_self ? 1 : 0;
  return s;
}

// dW[n, k] = sum_t a[t, n] b[t, k]: into the weight's gradient sink (accumulate) or a fresh tensor that is returned.
Spec wgrad_spec(const Tensor& a, const Tensor& b, const WTuple& w, std::vector<Tensor>& fresh, bool zero_fresh) {
  Spec s;
  s.a = a;
  s.a_mn = true;
  s.b = b;
  s.b_mn = true;
  if (has_sink(w)) {
    s.out = *std::get<1>(w);
    s.flags = wx::GEMM_ACCUMULATE;
    fresh.push_back(Tensor());
  } else {
    s.out = zero_fresh ? at::zeros_like(w_of(w)) : at::empty_like(w_of(w));
    fresh.push_back(s.out);
  }
  return s;
}

void check_common(const Tensor& x, const Tensor& cos_t, const Tensor& sin_t, const Tensor& qtab, const Tensor& ktab, int64_t d) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous(), "block: x must be contiguous CUDA bf16 [T, C]");
  TORCH_CHECK(cos_t.scalar_type() == at::kFloat && sin_t.scalar_type() == at::kFloat && cos_t.is_contiguous() && sin_t.is_contiguous() &&
                  cos_t.size(0) == x.size(0) && cos_t.size(1) == d,
              "block: cos/sin must be fp32 [T, head_dim]");
  TORCH_CHECK(qtab.scalar_type() == at::kInt && qtab.is_contiguous() && qtab.size(0) == x.size(0) && qtab.size(1) == 4 &&
                  ktab.scalar_type() == at::kInt && ktab.is_contiguous() && ktab.size(0) == x.size(0) && ktab.size(1) == 4,
              "block: attention tables must be int32 [T, 4]");
}

// Forward. `ffn` holds (gate_up, down) per expert: two entries for a dense FFN, 2 E for the dual-expert FFN (then
// dest / seg / inv / rows describe the token-type routing plan). Returns
// {out, y1, rstd1, qkv, o_attn, lse, x2, rstd2, xn, gu, h}: the result and what backward needs.
std::vector<Tensor> block_fwd(const Tensor& x, const Tensor& ln1_w, const WTuple& w_qkv, const OptT& b_qkv, const Tensor& cos_t,
                              const Tensor& sin_t, int64_t n_rot, const Tensor& qtab, const Tensor& ktab, int64_t hq, int64_t hkv,
                              int64_t d, double scale, bool has_bidir, const WTuple& w_o, const OptT& b_o, const Tensor& ln2_w,
                              double eps, const std::vector<WTuple>& ffn, const OptT& b_gu, const OptT& b_dn, const OptT& dest,
                              const OptT& seg, const OptT& inv, int64_t rows, bool need_bwd) {
  check_common(x, cos_t, sin_t, qtab, ktab, d);
  c10::cuda::CUDAGuard guard(x.device());
  int* status = wxb::status_tensor(x.device()).data_ptr<int>();
  const int64_t T = x.size(0), H = x.size(1);
  const bool moe = dest.has_value() && dest->defined();
  const int n_exp = static_cast<int>(ffn.size() / 2);
  TORCH_CHECK(ffn.size() >= 2 && ffn.size() % 2 == 0 && (moe || n_exp == 1), "block: ffn weights come in (gate_up, down) pairs");

  // ---- attention half
  auto [y1, rstd1] = norm_fwd(x, ln1_w, eps, OptT(), 0, false);
  Tensor qkv = empty_bf16(T, w_of(w_qkv).size(0), x);
  {
    std::vector<Spec> sp(1);
    sp[0].a = y1;
    sp[0].b = w_of(w_qkv);
    sp[0].out = qkv;
    sp[0].bias = b_qkv;
    launch(sp, {&w_qkv}, status);
  }
  rope_inplace(qkv, cos_t, sin_t, n_rot, d, false);
  Tensor o_attn = empty_bf16(T, hq * d, x);
  Tensor lse = at::empty({hq, T}, x.options().dtype(at::kFloat));
  {
    wx::AttnShape s = attn_shape(qkv, hq, hkv, d, scale, has_bidir, false);
    Tensor q = qkv.narrow(1, 0, hq * d), k = qkv.narrow(1, hq * d, hkv * d), v = qkv.narrow(1, (hq + hkv) * d, hkv * d);
    WX_RC(wx::attn_fwd(s, q.data_ptr(), k.data_ptr(), v.data_ptr(), qtab.data_ptr(), ktab.data_ptr(), o_attn.data_ptr(),
                       o_attn.stride(0), lse.data_ptr<float>(), cur(), status),
          "attn_fwd");
  }
  Tensor x2 = empty_bf16(T, H, x);
  {
    std::vector<Spec> sp(1);
    sp[0].a = o_attn;
    sp[0].b = w_of(w_o);
    sp[0].out = x2;
    sp[0].bias = b_o;
    sp[0].residual = x;
    launch(sp, {&w_o}, status);
  }

  // ---- FFN half
  Tensor out = empty_bf16(T, H, x), xn, rstd2, gu, h;
  if (moe) {
    std::tie(xn, rstd2) = norm_fwd(x2, ln2_w, eps, dest, rows, need_bwd);
    int64_t wmax = 0;
    for (int e = 0; e < n_exp; ++e) wmax = std::max<int64_t>(wmax, w_of(ffn[2 * e]).size(0));
    if (need_bwd) gu = empty_bf16(rows, wmax, x);
    h = empty_bf16(rows, wmax / 2, x);
    for (int e0 = 0; e0 < n_exp; e0 += 2) {
      std::vector<Spec> sp;
      std::vector<const WTuple*> ws;
      for (int e = e0; e < std::min(e0 + 2, n_exp); ++e) {
        Spec s;
        s.a = xn;
        s.b = w_of(ffn[2 * e]);
        s.out = h;
        if (need_bwd) s.out2 = gu;
        s.M = rows;
        s.dyn = seg->select(0, e);
        s.flags = wx::GEMM_ACT_SWIGLU | wx::GEMM_ZERO_PAD_ROWS;
        sp.push_back(s);
        ws.push_back(&ffn[2 * e]);
      }
      launch(sp, ws, status);
    }
    for (int e0 = 0; e0 < n_exp; e0 += 2) {
      std::vector<Spec> sp;
      std::vector<const WTuple*> ws;
      for (int e = e0; e < std::min(e0 + 2, n_exp); ++e) {
        const Tensor& w_dn = w_of(ffn[2 * e + 1]);
        Spec s;
        s.a = h.narrow(1, 0, w_dn.size(1));
        s.b = w_dn;
        s.out = out;
        s.M = rows;
        s.dyn = seg->select(0, e);
        s.row_map = inv;
        s.residual = x2;
        sp.push_back(s);
        ws.push_back(&ffn[2 * e + 1]);
      }
      launch(sp, ws, status);
    }
  } else {
    std::tie(xn, rstd2) = norm_fwd(x2, ln2_w, eps, OptT(), 0, false);
    const Tensor& w_gu = w_of(ffn[0]);
    const Tensor& w_dn = w_of(ffn[1]);
    if (need_bwd) gu = empty_bf16(T, w_gu.size(0), x);
    h = empty_bf16(T, w_gu.size(0) / 2, x);
    std::vector<Spec> sp(1);
    sp[0].a = xn;
    sp[0].b = w_gu;
    sp[0].out = h;
    if (need_bwd) sp[0].out2 = gu;
    sp[0].bias = b_gu;
    sp[0].flags = wx::GEMM_ACT_SWIGLU;
    launch(sp, {&ffn[0]}, status);
    std::vector<Spec> sd(1);
    sd[0].a = h;
    sd[0].b = w_dn;
    sd[0].out = out;
    sd[0].bias = b_dn;
    sd[0].residual = x2;
    launch(sd, {&ffn[1]}, status);
  }
  if (!need_bwd) return {out};
  return {out, y1, rstd1, qkv, o_attn, lse, x2, rstd2, xn, gu, h};
}

// Backward. Weight gradients go into the sinks (accumulate) where a weight has one; otherwise they are returned.
// Returns {dx, d ln1_w, d ln2_w, d b_qkv, d b_o, d b_gu, d b_dn, dW qkv, dW o, dW ffn[0], dW ffn[1], ...}
// with undefined tensors where nothing is due (no bias, or the gradient went into a sink).
std::vector<Tensor> block_bwd(const Tensor& dout_in, const Tensor& x, const Tensor& ln1_w, const Tensor& y1, const Tensor& rstd1,
                              const Tensor& qkv, const Tensor& o_attn, const Tensor& lse, const Tensor& x2, const Tensor& ln2_w,
                              const Tensor& rstd2, const Tensor& xn, const Tensor& gu, const Tensor& h, const WTuple& w_qkv,
                              bool has_b_qkv, const Tensor& cos_t, const Tensor& sin_t, int64_t n_rot, const Tensor& qtab,
                              const Tensor& ktab, int64_t hq, int64_t hkv, int64_t d, double scale, bool has_bidir, bool causal_self,
                              const WTuple& w_o, bool has_b_o, const std::vector<WTuple>& ffn, bool has_b_gu, bool has_b_dn,
                              const OptT& dest, const OptT& seg, const OptT& segk, int64_t rows, bool dn_in_place,
                              const std::vector<WTuple>& next_dn) {
  // dn_in_place: the down-projection weights are already whole in their staging views (the block whose backward ran
  // just before prefetched them); next_dn: up to two row-sharded weights to gather for the block whose backward runs
  // next (its down projections), carried by this block's last weight-gradient launch.
  check_common(x, cos_t, sin_t, qtab, ktab, d);
  c10::cuda::CUDAGuard guard(x.device());
  int* status = wxb::status_tensor(x.device()).data_ptr<int>();
  const int64_t T = x.size(0), H = x.size(1);
  const bool moe = dest.has_value() && dest->defined();
  const int n_exp = static_cast<int>(ffn.size() / 2);
  Tensor dout = dout_in.contiguous();
  // every weight row-sharded, and the two staging slots suffice (at most two experts): gathers ride on the wgrad GEMMs
  bool pf = prefetch_enabled() && n_exp <= 2 && gathered(w_qkv) && gathered(w_o) &&
            w_of(w_qkv).data_ptr() != w_of(w_o).data_ptr();
  for (const WTuple& w : ffn) pf = pf && gathered(w);
  if (pf && n_exp == 2)
    pf = w_of(ffn[0]).data_ptr() != w_of(ffn[2]).data_ptr() && w_of(ffn[1]).data_ptr() != w_of(ffn[3]).data_ptr();
  std::vector<Tensor> dW_ffn_dn, dW_ffn_gu, dW_o, dW_qkv;
  Tensor db_gu, db_dn, db_o, db_qkv;
  Tensor dxn;  // gradient w.r.t. the FFN's (normalised, possibly permuted) input

  // ---- FFN half
  if (moe) {
    Tensor dyp = at::zeros({rows, H}, x.options());  // grouped order, zero padding rows
    WX_RC(wx::permute_rows(dout.data_ptr(), dest->data_ptr<int>(), dyp.data_ptr(), T, H, cur(), static_cast<int>(rows)), "permute_rows");
    const int64_t wmax = gu.size(1);
    Tensor dgu = empty_bf16(rows, wmax, x);
    for (int e0 = 0; e0 < n_exp; e0 += 2) {  // dL/dh = dy @ w_down, turned into dL/d(gate|up) in the epilogue
      std::vector<Spec> sp;
      std::vector<const WTuple*> ws;
      for (int e = e0; e < std::min(e0 + 2, n_exp); ++e) {
        Spec s;
        s.a = dyp;
        s.b = w_of(ffn[2 * e + 1]);
        s.b_mn = true;
        s.out = dgu;
        s.out2 = gu;
        s.M = rows;
        s.dyn = seg->select(0, e);
        s.flags = wx::GEMM_SWIGLU_BWD | wx::GEMM_ZERO_PAD_ROWS;
        sp.push_back(s);
        ws.push_back(dn_in_place ? nullptr : &ffn[2 * e + 1]);
      }
      launch(sp, ws, status);
    }
    for (int e0 = 0; e0 < n_exp; e0 += 2) {  // dW_down[hid, i] over the expert's (128-padded) token segment
      std::vector<Spec> sp;
      for (int e = e0; e < std::min(e0 + 2, n_exp); ++e) {
        const int64_t I = w_of(ffn[2 * e + 1]).size(1);
        Spec s = wgrad_spec(dyp, h.narrow(1, 0, I), ffn[2 * e + 1], dW_ffn_dn, true);
        s.M = H;
        s.N = I;
        s.K = rows;
        s.dyn = segk->select(0, e);
        sp.push_back(s);
      }
      if (pf) {
        std::vector<const WTuple*> nxt;
        for (int e = 0; e < n_exp; ++e) nxt.push_back(&ffn[2 * e]);  // the gate/up weights, for the dgrad below
        launch_prefetching(sp, nxt, status);
      } else {
        launch(sp, std::vector<const WTuple*>(sp.size(), nullptr), status);
      }
    }
    dxn = empty_bf16(rows, H, x);
    for (int e0 = 0; e0 < n_exp; e0 += 2) {
      std::vector<Spec> sp;
      std::vector<const WTuple*> ws;
      for (int e = e0; e < std::min(e0 + 2, n_exp); ++e) {
        const Tensor& w_gu = w_of(ffn[2 * e]);
        Spec s;
        s.a = dgu.narrow(1, 0, w_gu.size(0));
        s.b = w_gu;
        s.b_mn = true;
        s.out = dxn;
        s.M = rows;
        s.dyn = seg->select(0, e);
        sp.push_back(s);
        ws.push_back(pf ? nullptr : &ffn[2 * e]);  // prefetched: already whole in its staging view
      }
      launch(sp, ws, status);
    }
    for (int e0 = 0; e0 < n_exp; e0 += 2) {
      std::vector<Spec> sp;
      for (int e = e0; e < std::min(e0 + 2, n_exp); ++e) {
        const int64_t W = w_of(ffn[2 * e]).size(0);
        Spec s = wgrad_spec(dgu.narrow(1, 0, W), xn, ffn[2 * e], dW_ffn_gu, true);
        s.M = W;
        s.N = H;
        s.K = rows;
        s.dyn = segk->select(0, e);
        sp.push_back(s);
      }
      if (pf) launch_prefetching(sp, {&w_o, &w_qkv}, status);  // for the two attention dgrads below
      else launch(sp, std::vector<const WTuple*>(sp.size(), nullptr), status);
    }
  } else {
    Tensor dgu = at::empty_like(gu);
    {
      std::vector<Spec> sp(1);
      sp[0].a = dout;
      sp[0].b = w_of(ffn[1]);
      sp[0].b_mn = true;
      sp[0].out = dgu;
      sp[0].out2 = gu;
      sp[0].flags = wx::GEMM_SWIGLU_BWD;
      launch(sp, {dn_in_place ? nullptr : &ffn[1]}, status);
    }
    {
      std::vector<Spec> sp{wgrad_spec(dout, h, ffn[1], dW_ffn_dn, false)};
      if (pf) launch_prefetching(sp, {&ffn[0]}, status);
      else launch(sp, {nullptr}, status);
    }
    if (has_b_dn) db_dn = col_sum(dout);
    dxn = empty_bf16(T, H, x);
    {
      std::vector<Spec> sp(1);
      sp[0].a = dgu;
      sp[0].b = w_of(ffn[0]);
      sp[0].b_mn = true;
      sp[0].out = dxn;
      launch(sp, {pf ? nullptr : &ffn[0]}, status);
    }
    {
      std::vector<Spec> sp{wgrad_spec(dgu, xn, ffn[0], dW_ffn_gu, false)};
      if (pf) launch_prefetching(sp, {&w_o, &w_qkv}, status);
      else launch(sp, {nullptr}, status);
    }
    if (has_b_gu) db_gu = col_sum(dgu);
  }
  auto [dx2, dln2] = norm_bwd(dxn, x2, ln2_w, rstd2, dest, dout);  // + gradient of the FFN's residual path
  dxn = Tensor();

  // ---- attention half
  Tensor d_oattn = at::empty_like(o_attn);
  {
    std::vector<Spec> sp(1);
    sp[0].a = dx2;
    sp[0].b = w_of(w_o);
    sp[0].b_mn = true;
    sp[0].out = d_oattn;
    launch(sp, {pf ? nullptr : &w_o}, status);
  }
  if (has_b_o) db_o = col_sum(dx2);
  Tensor dqkv = at::empty_like(qkv);
  {
    wx::AttnShape s = attn_shape(qkv, hq, hkv, d, scale, has_bidir, causal_self);
    Tensor q = qkv.narrow(1, 0, hq * d), k = qkv.narrow(1, hq * d, hkv * d), v = qkv.narrow(1, (hq + hkv) * d, hkv * d);
    Tensor dq = dqkv.narrow(1, 0, hq * d), dk = dqkv.narrow(1, hq * d, hkv * d), dv = dqkv.narrow(1, (hq + hkv) * d, hkv * d);
    auto fo = x.options().dtype(at::kFloat);
    Tensor delta = at::empty({hq, T}, fo);
    const int rep = static_cast<int>(hq / hkv);
    Tensor pk, pv;
    float *ppk = nullptr, *ppv = nullptr;
    if (rep > 1) {
      pk = at::empty({rep, T, hkv * d}, fo);
      pv = at::empty({rep, T, hkv * d}, fo);
      ppk = pk.data_ptr<float>();
      ppv = pv.data_ptr<float>();
    }
    WX_RC(wx::attn_bwd(s, q.data_ptr(), k.data_ptr(), v.data_ptr(), o_attn.data_ptr(), o_attn.stride(0), d_oattn.data_ptr(),
                       d_oattn.stride(0), lse.data_ptr<float>(), qtab.data_ptr(), ktab.data_ptr(), delta.data_ptr<float>(),
                       dq.data_ptr(), dq.stride(0), dk.data_ptr(), dk.stride(0), dv.data_ptr(), dv.stride(0), ppk, ppv, cur(), status),
          "attn_bwd");
    g_launches.fetch_add(rep > 1 ? 4 : 2, std::memory_order_relaxed);  // delta, dQ, dK/dV (+ the two partial reductions)
  }
  d_oattn = Tensor();
  rope_inplace(dqkv, cos_t, sin_t, n_rot, d, true);
  Tensor& dqkv_raw = dqkv;
  Tensor dy1 = empty_bf16(T, H, x);
  {
    std::vector<Spec> sp(1);
    sp[0].a = dqkv_raw;
    sp[0].b = w_of(w_qkv);
    sp[0].b_mn = true;
    sp[0].out = dy1;
    launch(sp, {pf ? nullptr : &w_qkv}, status);
  }
  {
    // the two attention weight gradients share one launch: each alone leaves most of its last wave of tiles idle
    // (weights of a few thousand rows and columns give barely more tiles than SMs), together they fill it
    std::vector<Spec> sp{wgrad_spec(dqkv_raw, y1, w_qkv, dW_qkv, false), wgrad_spec(dx2, o_attn, w_o, dW_o, false)};
    if (!next_dn.empty()) {
      std::vector<const WTuple*> nxt;
      for (const WTuple& w : next_dn) nxt.push_back(&w);
      launch_prefetching(sp, nxt, status);
    } else {
      launch(sp, {nullptr, nullptr}, status);
    }
  }
  if (has_b_qkv) db_qkv = col_sum(dqkv_raw);
  auto [dx, dln1] = norm_bwd(dy1, x, ln1_w, rstd1, OptT(), dx2);  // + gradient of the attention's residual path

  std::vector<Tensor> res{dx, dln1, dln2, db_qkv, db_o, db_gu, db_dn, dW_qkv[0], dW_o[0]};
  for (int e = 0; e < n_exp; ++e) {
    res.push_back(dW_ffn_gu[e]);
    res.push_back(dW_ffn_dn[e]);
  }
  return res;
}

}  // namespace

void register_block_bindings(pybind11::module_& m) {
  m.def("block_fwd", &block_fwd, "one pre-norm attention + FFN block, forward: every kernel enqueued by one host call");
  m.def("block_bwd", &block_bwd, "backward of block_fwd");
  m.def("block_launch_count", []() { return g_launches.load(); }, "kernels launched by block_fwd / block_bwd so far");
}

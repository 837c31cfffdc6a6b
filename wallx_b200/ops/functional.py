"""Differentiable operator API used by the model code.

Dispatch rule (no multi-backend layer): a CUDA tensor runs the hand-written sm_100a kernels of the
in-tree extension and raises if the extension is missing; a CPU tensor runs the PyTorch oracle in
:mod:`wallx_b200.ops.ref`.

Layouts are B200-first rather than the reference's: activations are token-packed ``[T, C]`` (no
padding rows), q/k/v live in one ``[T, (Hq + 2 Hkv) * D]`` buffer written by one fused GEMM, FFN
gate/up weights are interleaved in 16-row blocks so SwiGLU runs in the GEMM epilogue, and expert
routing uses 128-row aligned segments so that forward, dgrad and wgrad are all tile-aligned.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Sequence, Tuple

import torch

from . import ref
from . import gemm as G
from . import _ext


def _is_cuda(x: torch.Tensor) -> bool:
    return x.is_cuda


def _C():
    return _ext.get()


# Gradient sinks: when a weight lives in a flat gradient buffer, its weight-gradient GEMM adds
# straight into that buffer (GEMM epilogue with the accumulate flag) instead of producing a
# temporary that autograd then adds: one kernel and one pass over the gradient less per weight.
# The sink is an attribute of the parameter object: ``(gradient view, callback, data pointer at
# registration)``. Row-sharded parameters share a staging buffer, so an address cannot name them;
# for them the pointer entry is None.
_SINK_OWNERS = None


def register_grad_sink(weight: torch.Tensor, grad_view: torch.Tensor, mark) -> None:
    import weakref

    global _SINK_OWNERS
    if _SINK_OWNERS is None:
        _SINK_OWNERS = weakref.WeakSet()
    weight._wx_sink = (grad_view, mark, weight.data_ptr())
    _SINK_OWNERS.add(weight)


def _sink_of(w: torch.Tensor):
    s = getattr(w, "_wx_sink", None)
    if s is None:
        return None
    moved = getattr(w, "_wx_shard", None) is None and s[2] != w.data_ptr()  # .to() / .data re-pointed since registration
    if moved or s[0].shape != w.shape or s[0].device != w.device or not _pitch_ok(s[0]):
        return None
    return s


def clear_grad_sinks() -> None:
    if _SINK_OWNERS is not None:
        for w in list(_SINK_OWNERS):
            if hasattr(w, "_wx_sink"):
                del w._wx_sink
        _SINK_OWNERS.clear()


def _shard_of(w: torch.Tensor):
    """The fused-gather record of a row-sharded weight (``parallel/zero3.py``), or None for a resident one."""
    return getattr(w, "_wx_shard", None)


def _launch(specs, weights) -> None:
    """Launch one or two problems whose B operands are ``weights``. Resident weights take the plain GEMM; a
    row-sharded weight is gathered from its owners inside the launch (two sharded weights share a launch when
    they sit in different staging slots)."""
    shards = [_shard_of(w) for w in weights]
    if all(s is None for s in shards):
        G.launch(specs)
        return
    from ..parallel.ag_linear import ag_launch

    if all(s is not None for s in shards) and (len(shards) == 1 or shards[0].slot != shards[1].slot):
        ag_launch(specs, shards)
        return
    for spec, s in zip(specs, shards):
        if s is None:
            G.launch([spec])
        else:
            ag_launch([spec], [s])


def _wgrad(a: torch.Tensor, b: torch.Tensor, w: torch.Tensor, **spec_kw):
    """dW[n, k] = sum_t a[t, n] b[t, k] (+ optional dyn/K overrides). Returns the gradient to hand
    to autograd, or None when it was accumulated into the weight's sink."""
    sink = _sink_of(w)
    if sink is not None:
        G.launch([G.GemmSpec(a, b, sink[0], a_mn=True, b_mn=True, flags=G.ACCUMULATE, **spec_kw)])
        sink[1]()
        return None
    dw = torch.zeros_like(w) if "dyn" in spec_kw else torch.empty_like(w)
    G.launch([G.GemmSpec(a, b, dw, a_mn=True, b_mn=True, **spec_kw)])
    return dw


def _pitch_ok(t: torch.Tensor) -> bool:
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def _aligned2d(t: torch.Tensor) -> torch.Tensor:
    """Return ``t`` or a copy whose row pitch is a multiple of 16 bytes (view of a padded buffer)."""
    if _pitch_ok(t):
        return t
    rows, cols = t.shape
    pc = (cols + 7) // 8 * 8
    buf = torch.zeros((rows, pc), device=t.device, dtype=t.dtype)
    buf[:, :cols].copy_(t)
    return buf[:, :cols]


# ----------------------------------------------------------------------------- linear
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, residual):
        x2 = _aligned2d(x)
        w2 = _aligned2d(w)
        out = torch.empty((x.shape[0], w.shape[0]), device=x.device, dtype=torch.bfloat16)
        _launch([G.GemmSpec(x2, w2, out, bias=b, residual=residual)], [w2])
        ctx.save_for_backward(x, w)
        ctx.has_bias = b is not None
        ctx.has_res = residual is not None
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dy2 = _aligned2d(dy)
        dx = dw = db = dres = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            # dx[m, k] = sum_n dy[m, n] w[n, k]: B(n'=k, k'=n) is w read as MN-major
            w2 = _aligned2d(w)
            _launch([G.GemmSpec(dy2, w2, dx, b_mn=True)], [w2])
        if ctx.needs_input_grad[1]:
            # dw[n, k] = sum_m dy[m, n] x[m, k]: both operands MN-major over the token axis
            dw = _wgrad(dy2, _aligned2d(x), w)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = column_sum(dy)
        if ctx.has_res and ctx.needs_input_grad[3]:
            dres = dy
        return dx, dw, db, dres


def column_sum(x: torch.Tensor) -> torch.Tensor:
    """Sum over rows of a ``[R, C]`` tensor in fp32, returned in x's dtype (bias gradients)."""
    if _is_cuda(x) and x.dtype == torch.bfloat16:
        return _C().column_sum(x.contiguous())
    return x.float().sum(0).to(x.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T + b (+ residual)`` over the last dimension; residual add is fused on CUDA."""
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    if _is_cuda(x2):
        if x2.dtype != torch.bfloat16:
            raise TypeError("CUDA path is bf16; cast the model and inputs to bfloat16")
        r2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        if r2 is not None and not (r2.stride(1) == 1):
            r2 = r2.contiguous()
        y = _LinearFn.apply(x2 if x2.stride(1) == 1 else x2.contiguous(), w, b, r2)
    else:
        y = ref.linear(x2, w, b)
        if residual is not None:
            y = y + residual.reshape(-1, w.shape[0])
    return y.reshape(*shp[:-1], w.shape[0])


def linear_gelu(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    """``gelu(x @ w.T + b)`` (exact erf GELU). Fused into the GEMM epilogue when no grad is needed."""
    if _is_cuda(x) and not (torch.is_grad_enabled() and (x.requires_grad or w.requires_grad)):
        x2 = _aligned2d(x.reshape(-1, x.shape[-1]))
        out = torch.empty((x2.shape[0], w.shape[0]), device=x.device, dtype=torch.bfloat16)
        w2 = _aligned2d(w)
        _launch([G.GemmSpec(x2, w2, out, bias=b, flags=G.ACT_GELU)], [w2])
        return out.reshape(*x.shape[:-1], w.shape[0])
    return torch.nn.functional.gelu(linear(x, w, b))


# ----------------------------------------------------------------------------- RMSNorm
class _RmsNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, dest, out_rows):
        # rows that no token maps to must be zero only when a backward pass will reduce over them
        y, rstd = _C().rms_norm_fwd(x, w, float(eps), dest, int(out_rows), bool(any(ctx.needs_input_grad)))
        ctx.save_for_backward(x, w, rstd, dest if dest is not None else torch.empty(0))
        ctx.has_dest = dest is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd, dest = ctx.saved_tensors
        dx, dw = _C().rms_norm_bwd(dy.contiguous(), x, w, rstd, dest if ctx.has_dest else None)
        return dx, dw, None, None, None


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, dest: Optional[torch.Tensor] = None,
             out_rows: int = 0) -> torch.Tensor:
    """RMSNorm over the last dimension (fp32 statistics).

    With ``dest`` (int32 ``[T]``) row ``t`` of the result is written to row ``dest[t]`` of a
    zero-filled ``[out_rows, C]`` buffer: the token-type permutation of the expert FFN is fused
    into the normalisation that precedes it.
    """
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    if _is_cuda(x2):
        y = _RmsNormFn.apply(x2.contiguous(), w, eps, dest, out_rows)
        return y if dest is not None else y.reshape(shp)
    y = ref.rms_norm(x2, w, eps)
    if dest is not None:
        return ref.permute_rows(y, dest.long(), out_rows)
    return y.reshape(shp)


# ----------------------------------------------------------------------------- SwiGLU FFN pieces
class _GateUpFn(torch.autograd.Function):
    """h = silu(g) * u with [g | u] = x @ w_gu.T (+ b) interleaved in 16-column blocks."""

    @staticmethod
    def forward(ctx, x, w_gu, b_gu):
        M, N = x.shape[0], w_gu.shape[0]
        # the raw gate/up values are only needed by the backward pass
        gu = torch.empty((M, N), device=x.device, dtype=torch.bfloat16) if any(ctx.needs_input_grad) else None
        h = torch.empty((M, N // 2), device=x.device, dtype=torch.bfloat16)
        _launch([G.GemmSpec(x, w_gu, h, out2=gu, bias=b_gu, flags=G.ACT_SWIGLU)], [w_gu])
        if gu is not None:
            ctx.save_for_backward(x, w_gu, gu)
        ctx.has_bias = b_gu is not None
        return h

    @staticmethod
    def backward(ctx, dh):
        x, w_gu, gu = ctx.saved_tensors
        dgu = _C().swiglu_bwd(dh.contiguous(), gu)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            _launch([G.GemmSpec(dgu, w_gu, dx, b_mn=True)], [w_gu])
        if ctx.needs_input_grad[1]:
            dw = _wgrad(dgu, x, w_gu)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = column_sum(dgu)
        return dx, dw, db


# SwiGLU backward inside the down-projection's dgrad epilogue (dL/dh never goes to memory) or as a separate
# streaming kernel after a plain dgrad GEMM. Both are kept: which one is faster depends on how far the GEMM is
# from being epilogue-bound (environment variable WX_FUSE_SWIGLU_BWD=0/1).
FUSE_SWIGLU_BWD = os.environ.get("WX_FUSE_SWIGLU_BWD", "1") != "0"


class _SwiGLUFfnFn(torch.autograd.Function):
    """Whole SwiGLU FFN, ``down(silu(gate(x)) * up(x)) (+ bias) (+ residual)``, as one autograd node so
    that the backward of the activation runs in the epilogue of the down-projection's dgrad GEMM:
    ``dL/dh`` never goes to memory."""

    @staticmethod
    def forward(ctx, x, w_gu, b_gu, w_dn, b_dn, residual):
        M, N = x.shape[0], w_gu.shape[0]
        need_bwd = any(ctx.needs_input_grad)
        gu = torch.empty((M, N), device=x.device, dtype=torch.bfloat16) if need_bwd else None
        h = torch.empty((M, N // 2), device=x.device, dtype=torch.bfloat16)
        _launch([G.GemmSpec(x, w_gu, h, out2=gu, bias=b_gu, flags=G.ACT_SWIGLU)], [w_gu])
        out = torch.empty((M, w_dn.shape[0]), device=x.device, dtype=torch.bfloat16)
        _launch([G.GemmSpec(h, w_dn, out, bias=b_dn, residual=residual)], [w_dn])
        if need_bwd:
            ctx.save_for_backward(x, w_gu, w_dn, gu, h)
        ctx.has_bgu, ctx.has_bdn, ctx.has_res = b_gu is not None, b_dn is not None, residual is not None
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w_gu, w_dn, gu, h = ctx.saved_tensors
        dy = dy.contiguous()
        if FUSE_SWIGLU_BWD:
            dgu = torch.empty_like(gu)
            # dL/dh = dy @ w_dn, turned into dL/d(gate|up) in the epilogue
            _launch([G.GemmSpec(dy, w_dn, dgu, b_mn=True, out2=gu, flags=G.SWIGLU_BWD)], [w_dn])
        else:
            dh = torch.empty_like(h)
            _launch([G.GemmSpec(dy, w_dn, dh, b_mn=True)], [w_dn])
            dgu = _C().swiglu_bwd(dh, gu)
        dx = dw_gu = db_gu = dw_dn = db_dn = dres = None
        if ctx.needs_input_grad[3]:
            dw_dn = _wgrad(dy, h, w_dn)
        if ctx.has_bdn and ctx.needs_input_grad[4]:
            db_dn = column_sum(dy)
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            _launch([G.GemmSpec(dgu, w_gu, dx, b_mn=True)], [w_gu])
        if ctx.needs_input_grad[1]:
            dw_gu = _wgrad(dgu, x, w_gu)
        if ctx.has_bgu and ctx.needs_input_grad[2]:
            db_gu = column_sum(dgu)
        if ctx.has_res and ctx.needs_input_grad[5]:
            dres = dy
        return dx, dw_gu, db_gu, dw_dn, db_dn, dres


def swiglu_ffn(x: torch.Tensor, w_gu: torch.Tensor, b_gu: Optional[torch.Tensor], w_dn: torch.Tensor,
               b_dn: Optional[torch.Tensor], residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``down(silu(gate(x)) * up(x)) + b (+ residual)`` with ``w_gu [2I, K]`` interleaved in 16-row blocks.
    Reference: Qwen2_5_VLMLP / Qwen2MLP (modeling_qwen2_5_vl.py:357-363, 715-728) as three cuBLAS GEMMs and
    unfused elementwise kernels."""
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    if _is_cuda(x2):
        r2 = residual.reshape(-1, w_dn.shape[0]) if residual is not None else None
        if r2 is not None and r2.stride(1) != 1:
            r2 = r2.contiguous()
        y = _SwiGLUFfnFn.apply(x2.contiguous(), w_gu, b_gu, w_dn, b_dn, r2)
        return y.reshape(*shp[:-1], w_dn.shape[0])
    h = gate_up_swiglu(x, w_gu, b_gu)
    return linear(h, w_dn, b_dn, residual)


def gate_up_swiglu(x: torch.Tensor, w_gu: torch.Tensor, b_gu: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Fused gate/up projection + SwiGLU; ``w_gu`` is ``[2I, K]`` interleaved in 16-row blocks."""
    x2 = x.reshape(-1, x.shape[-1])
    if _is_cuda(x2):
        h = _GateUpFn.apply(x2.contiguous(), w_gu, b_gu)
    else:
        h = ref.swiglu_interleaved(ref.linear(x2, w_gu, b_gu))
    return h.reshape(*x.shape[:-1], w_gu.shape[0] // 2)


# ----------------------------------------------------------------------------- dual-expert FFN
class RoutePlan:
    """Grouping of tokens by expert (token type) for one batch; shared by every decoder layer.

    ``dest`` int32 ``[T]``: row of each token in the grouped buffer (segment starts are multiples of
    128 rows). ``seg`` int32 ``[E, 4]`` = ``(start, count, -1, -1)`` and ``segk`` = ``(-1, -1, start,
    padded_count)`` live on the device and are read by the grouped GEMM directly (row-segment
    problems and reductions over a segment), so no launch needs host-side sizes. ``inv`` int32
    ``[rows]`` maps a grouped row back to its token (-1 on padding rows). ``rows`` is the host-side
    upper bound of the grouped buffer height.
    """

    @staticmethod
    def note_single_expert(plan: "Optional[RoutePlan]", token_types: torch.Tensor) -> None:
        """Record on ``plan`` that all of ``token_types`` are equal (one host read; call outside hot loops)."""
        if plan is None or token_types.numel() == 0:
            return
        t = token_types.reshape(-1)
        first = int(t[0])
        if bool((t == first).all()):
            plan.single_expert = first

    def __init__(self, dest, seg, segk, inv, rows: int):
        self.dest, self.seg, self.segk, self.inv, self.rows = dest, seg, segk, inv, rows
        # set by a caller that knows on the host that every token goes to one expert (the action rows of a denoise
        # step, the text tokens of a decoding step): inference paths then run that expert as a plain FFN, without
        # grouping rows
        self.single_expert: Optional[int] = None


def route_rows(T: int, num_experts: int) -> int:
    return (T + 127) // 128 * 128 + 128 * (num_experts - 1)


def make_route_plan(token_types: torch.Tensor, num_experts: int) -> RoutePlan:
    """Build the plan. On CUDA this is one kernel (ballot + prefix count per expert id) and no host
    sync: the buffer height is bounded by ``round_up(T, 128) + 128 (E - 1)``.

    Replaces the reference's radix sort + row-map kernels (csrc/permute.cu:39-67, 450-494) and the
    per-expert ``.sum()`` host syncs (modeling_qwen2_5_vl_act.py:1275-1283).
    """
    tt = token_types.reshape(-1)
    T = tt.numel()
    rows = route_rows(T, num_experts)
    if _is_cuda(tt):
        dest, seg, segk, inv = _C().route_plan(tt.to(torch.int32).contiguous(), int(num_experts), int(rows))
        return RoutePlan(dest, seg, segk, inv, rows)
    dest, seg3 = ref.route_plan(tt, num_experts, 128)
    neg = torch.full_like(seg3[:, 0], -1)
    seg = torch.stack([seg3[:, 0], seg3[:, 1], neg, neg], dim=1).to(torch.int32)
    segk = torch.stack([neg, neg, seg3[:, 0], seg3[:, 2]], dim=1).to(torch.int32)
    inv = torch.full((rows,), -1, dtype=torch.int32)
    inv[dest] = torch.arange(T, dtype=torch.int32)
    return RoutePlan(dest.to(torch.int32), seg, segk, inv, rows)


class _MoeFfnFn(torch.autograd.Function):
    """Grouped gate/up+SwiGLU, then grouped down-projection with the un-permute (row scatter) and
    the residual add fused into its epilogue. Two problems (experts) per launch."""

    @staticmethod
    def forward(ctx, xp, residual, dest, seg, segk, inv, n_exp, *weights):
        # weights = (w_gu_0, w_down_0, w_gu_1, w_down_1, ...)
        rows, H = xp.shape
        T = dest.numel()
        wmax = max(weights[2 * e].shape[0] for e in range(n_exp))
        # the raw gate/up values are only needed by the backward pass
        gu = torch.empty((rows, wmax), device=xp.device, dtype=torch.bfloat16) if any(ctx.needs_input_grad) else None
        h = torch.empty((rows, wmax // 2), device=xp.device, dtype=torch.bfloat16)
        out = torch.empty((T, H), device=xp.device, dtype=torch.bfloat16)
        specs = [G.GemmSpec(xp, weights[2 * e], h, out2=gu, M=rows, dyn=seg[e],
                            flags=G.ACT_SWIGLU | G.ZERO_PAD_ROWS) for e in range(n_exp)]
        for i in range(0, n_exp, 2):
            _launch(specs[i:i + 2], [weights[2 * e] for e in range(i, min(i + 2, n_exp))])
        specs = []
        for e in range(n_exp):
            w_dn = weights[2 * e + 1]
            specs.append(G.GemmSpec(h[:, : w_dn.shape[1]], w_dn, out, M=rows, dyn=seg[e], row_map=inv,
                                    residual=residual))
        for i in range(0, n_exp, 2):
            _launch(specs[i:i + 2], [weights[2 * e + 1] for e in range(i, min(i + 2, n_exp))])
        if gu is not None:
            ctx.save_for_backward(xp, dest, seg, segk, gu, h, *weights)
        ctx.n_exp = n_exp
        ctx.has_res = residual is not None
        return out

    @staticmethod
    def backward(ctx, dout):
        xp, dest, seg, segk, gu, h, *weights = ctx.saved_tensors
        n_exp = ctx.n_exp
        rows, H = xp.shape
        dout = dout.contiguous()
        dyp = _C().permute_rows(dout, dest, rows)  # grouped order, zero padding rows
        wmax = gu.shape[1]
        # dL/dh = dy @ w_down per expert, turned into dL/d(gate|up) in the GEMM epilogue (pad rows zeroed)
        specs = []
        if FUSE_SWIGLU_BWD:
            dgu = torch.empty((rows, wmax), device=xp.device, dtype=torch.bfloat16)
            for e in range(n_exp):
                w_dn = weights[2 * e + 1]
                specs.append(G.GemmSpec(dyp, w_dn, dgu, M=rows, dyn=seg[e], b_mn=True, out2=gu,
                                        flags=G.SWIGLU_BWD | G.ZERO_PAD_ROWS))
            for i in range(0, n_exp, 2):
                _launch(specs[i:i + 2], [weights[2 * e + 1] for e in range(i, min(i + 2, n_exp))])
        else:
            dh = torch.empty((rows, wmax // 2), device=xp.device, dtype=torch.bfloat16)
            for e in range(n_exp):
                w_dn = weights[2 * e + 1]
                specs.append(G.GemmSpec(dyp, w_dn, dh[:, : w_dn.shape[1]], M=rows, dyn=seg[e], b_mn=True,
                                        flags=G.ZERO_PAD_ROWS))
            for i in range(0, n_exp, 2):
                _launch(specs[i:i + 2], [weights[2 * e + 1] for e in range(i, min(i + 2, n_exp))])
            dgu = _C().swiglu_bwd(dh, gu)
        grads = [None] * (2 * n_exp)
        specs = []
        marks = []  # sink callbacks run once the GEMM that adds into the sink has been enqueued
        for e in range(n_exp):
            w_dn = weights[2 * e + 1]
            I = w_dn.shape[1]
            sink = _sink_of(w_dn)
            if sink is not None:  # accumulate straight into the flat gradient buffer
                dw, fl = sink[0], G.ACCUMULATE
                marks.append(sink[1])
            else:
                dw, fl = torch.zeros_like(w_dn), 0  # stays zero when the expert has no tokens
                grads[2 * e + 1] = dw
            # dw[hid, i] = sum over the expert's (128-padded) token segment of dy[t, hid] h[t, i]
            specs.append(G.GemmSpec(dyp, h[:, :I], dw, a_mn=True, b_mn=True, M=H, N=I, K=rows, dyn=segk[e], flags=fl))
        for i in range(0, n_exp, 2):
            G.launch(specs[i:i + 2])
        for mark in marks:
            mark()
        dxp = torch.empty((rows, H), device=xp.device, dtype=torch.bfloat16)
        specs = []
        for e in range(n_exp):
            w_gu = weights[2 * e]
            specs.append(G.GemmSpec(dgu[:, : w_gu.shape[0]], w_gu, dxp, M=rows, dyn=seg[e], b_mn=True))
        for i in range(0, n_exp, 2):
            _launch(specs[i:i + 2], [weights[2 * e] for e in range(i, min(i + 2, n_exp))])
        specs = []
        marks = []
        for e in range(n_exp):
            w_gu = weights[2 * e]
            W = w_gu.shape[0]
            sink = _sink_of(w_gu)
            if sink is not None:
                dw, fl = sink[0], G.ACCUMULATE
                marks.append(sink[1])
            else:
                dw, fl = torch.zeros_like(w_gu), 0
                grads[2 * e] = dw
            specs.append(G.GemmSpec(dgu[:, :W], xp, dw, a_mn=True, b_mn=True, M=W, N=H, K=rows, dyn=segk[e], flags=fl))
        for i in range(0, n_exp, 2):
            G.launch(specs[i:i + 2])
        for mark in marks:
            mark()
        dres = dout if ctx.has_res else None
        return (dxp, dres, None, None, None, None, None, *grads)


def moe_ffn(xp: torch.Tensor, residual: Optional[torch.Tensor], plan: RoutePlan,
            weights: Sequence[Tuple[torch.Tensor, torch.Tensor]]) -> torch.Tensor:
    """Token-type-routed expert FFN on a grouped input.

    ``xp`` ``[rows, H]`` is the grouped (permuted, zero-padded) input produced by
    :func:`rms_norm` with ``dest=plan.dest``; ``weights[e] = (w_gate_up_interleaved [2 I_e, H],
    w_down [H, I_e])``. Returns ``residual + ffn(x)`` in token order ``[T, H]``.

    Reference path replaced: permute -> per-expert 3x cuBLAS loop -> unpermute
    (modeling_qwen2_5_vl_act.py:138-157) and the dormant CUTLASS grouped GEMM
    (fusions/ops.py:6-165).
    """
    n_exp = len(weights)
    if _is_cuda(xp):
        flat = []
        for wg, wd in weights:
            flat += [wg, wd]
        return _MoeFfnFn.apply(xp, residual, plan.dest, plan.seg, plan.segk, plan.inv, n_exp, *flat)
    T = plan.dest.numel()
    out_p = torch.zeros_like(xp)
    seg = plan.seg.tolist()
    for e, (wg, wd) in enumerate(weights):
        s, c = seg[e][0], seg[e][1]
        if c == 0:
            continue
        he = ref.swiglu_interleaved(ref.linear(xp[s:s + c], wg))
        out_p = out_p.clone()
        out_p[s:s + c] = ref.linear(he, wd)
    y = ref.unpermute_rows(out_p, plan.dest.long())
    return y + residual if residual is not None else y


# ----------------------------------------------------------------------------- rotary
class _RopeQkFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, n_rot_heads, head_dim):
        out = _C().rope_qk(qkv, cos, sin, int(n_rot_heads), int(head_dim), False)
        ctx.save_for_backward(cos, sin)
        ctx.n_rot_heads, ctx.head_dim = n_rot_heads, head_dim
        return out

    @staticmethod
    def backward(ctx, dout):
        cos, sin = ctx.saved_tensors
        dqkv = _C().rope_qk(dout.contiguous(), cos, sin, int(ctx.n_rot_heads), int(ctx.head_dim), True)
        return dqkv, None, None, None, None


def rope_qk(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot_heads: int, head_dim: int) -> torch.Tensor:
    """Rotate the first ``n_rot_heads`` heads (q then k) of a packed ``[T, heads*D]`` buffer;
    the remaining (v) columns are copied. cos/sin are fp32 ``[T, D]`` (rotate-half form).

    Replaces csrc/rope.cu:48-330 (forward and backward share one kernel here: the backward is the
    inverse rotation)."""
    if _is_cuda(qkv):
        return _RopeQkFn.apply(qkv.contiguous(), cos, sin, n_rot_heads, head_dim)
    T = qkv.shape[0]
    rot = qkv[:, : n_rot_heads * head_dim].reshape(T, n_rot_heads, head_dim)
    rot = ref.apply_rope(rot, cos, sin).reshape(T, -1)
    return torch.cat([rot, qkv[:, n_rot_heads * head_dim:]], dim=-1)


# ----------------------------------------------------------------------------- attention
class AttnMeta:
    """Host-side description of the packed sequences of one attention call.

    Queries and keys may live in different buffers with different per-sequence lengths (prefix
    reuse: few new queries against a long cached key range). The causal rule is bottom-right
    aligned: query ``i`` of a sequence sees keys ``j <= i + (Lk - Lq)``; in addition a query
    flagged in ``bidir_q`` sees every key flagged in ``bidir_k`` (the action-token block).
    """

    def __init__(self, cu_q: Sequence[int], device, causal: bool, bidir_q: Optional[torch.Tensor] = None,
                 cu_k: Optional[Sequence[int]] = None, bidir_k: Optional[torch.Tensor] = None,
                 cache_rows: Optional[torch.Tensor] = None, k_starts: Optional[Sequence[int]] = None,
                 k_lens: Optional[Sequence[int]] = None, k_rows: Optional[int] = None):
        """Key ranges are either ``cu_k`` (adjacent segments), or ``k_starts``/``k_lens`` (one
        range per sequence inside a larger buffer of ``k_rows`` rows, e.g. KV-cache slots), or
        absent (self-attention: keys are the queries' own rows)."""
        self.cu_q_host = [int(c) for c in cu_q]
        nseq = len(self.cu_q_host) - 1
        self.self_attn = cu_k is None and k_starts is None
        if k_starts is not None:
            self.k_ranges = [(int(s0), int(s0) + int(l)) for s0, l in zip(k_starts, k_lens)]
            self.k_rows = int(k_rows) if k_rows is not None else max(e for _, e in self.k_ranges)
        else:
            ck = [int(c) for c in cu_k] if cu_k is not None else self.cu_q_host
            self.k_ranges = [(ck[i], ck[i + 1]) for i in range(nseq)]
            self.k_rows = ck[-1]
        self.cu_k_host = [r[0] for r in self.k_ranges] + [self.k_ranges[-1][1] if self.k_ranges else 0]
        self.cu_q = torch.tensor(self.cu_q_host, dtype=torch.int32, device=device)
        lq = [self.cu_q_host[i + 1] - self.cu_q_host[i] for i in range(nseq)]
        lk = [e - s0 for s0, e in self.k_ranges]
        self.max_q = max(lq) if lq else 0
        self.max_k = max(lk) if lk else 0
        self.causal = bool(causal)
        self.bidir_q = bidir_q
        self.bidir_k = bidir_k if bidir_k is not None else (bidir_q if self.self_attn else None)
        self.cache_rows = cache_rows
        self._dev = {}

    # legacy names used by the packed self-attention path
    @property
    def cu_host(self):
        return self.cu_q_host

    def device_tables(self, device):
        """Per-token tables for the kernels: for every query row its key range and causal limit."""
        t = self._dev.get("tables")
        if t is None:
            nq, nk = self.cu_q_host[-1], self.k_rows
            k_lo = torch.zeros(nq, dtype=torch.int32)
            k_hi = torch.zeros(nq, dtype=torch.int32)
            k_lim = torch.full((nq,), -1, dtype=torch.int32)  # last visible key (absolute row) under causality
            q_lo = torch.zeros(nk, dtype=torch.int32)
            q_hi = torch.zeros(nk, dtype=torch.int32)
            q_first = torch.zeros(nk, dtype=torch.int32)  # first query row that sees the key (causal rule)
            seq_of_q = torch.zeros(nq, dtype=torch.int64)
            seq_of_k = torch.zeros(nk, dtype=torch.int64)
            for b in range(len(self.cu_q_host) - 1):
                q0, q1 = self.cu_q_host[b], self.cu_q_host[b + 1]
                k0, k1 = self.k_ranges[b]
                k_lo[q0:q1] = k0
                k_hi[q0:q1] = k1
                off = (k1 - k0) - (q1 - q0)
                k_lim[q0:q1] = torch.arange(q1 - q0, dtype=torch.int32) + (k0 + off)
                q_lo[k0:k1] = q0
                q_hi[k0:k1] = q1
                q_first[k0:k1] = (torch.arange(k1 - k0, dtype=torch.int32) - off).clamp_(min=0) + q0 if self.causal else q0
                seq_of_q[q0:q1] = b
                seq_of_k[k0:k1] = b
            if not self.causal:
                k_lim = k_hi - 1
            # flags stay on their device (no host round trip); host-built columns are uploaded once
            qh = torch.stack([k_lo, k_hi, k_lim], dim=1).to(device, non_blocking=True)
            kh = torch.stack([q_lo, q_hi], dim=1).to(device, non_blocking=True)
            qc = q_first.to(device, non_blocking=True)  # first viewer under the causal rule
            qf = qc
            fq = (self.bidir_q.to(device=device, dtype=torch.int32) if self.bidir_q is not None
                  else torch.zeros(nq, dtype=torch.int32, device=device))
            fk = (self.bidir_k.to(device=device, dtype=torch.int32) if self.bidir_k is not None
                  else torch.zeros(nk, dtype=torch.int32, device=device))
            if self.causal and self.bidir_q is not None and self.bidir_k is not None:
                # a flagged key is also seen by every flagged query of its sequence: the first one
                nseq = len(self.cu_q_host) - 1
                rows = torch.arange(nq, dtype=torch.int32, device=device)
                cand = torch.where(fq > 0, rows, torch.full_like(rows, nq))
                first = torch.full((nseq,), nq, dtype=torch.int32, device=device)
                first = first.scatter_reduce(0, seq_of_q.to(device), cand, reduce="amin", include_self=True)
                per_key = first.index_select(0, seq_of_k.to(device))
                qf = torch.where(fk > 0, torch.minimum(qc, per_key), qc)
            else:
                fq = torch.zeros_like(fq)
                fk = torch.zeros_like(fk)
            qtab = torch.cat([qh, fq.reshape(-1, 1)], dim=1).contiguous()
            ktab = torch.cat([kh, qc.reshape(-1, 1), (fk + 2 * qf).reshape(-1, 1)], dim=1).contiguous()
            t = (qtab, ktab)
            self._dev["tables"] = t
        return t


def _attention_torch(q, k, v, meta: AttnMeta, hq, hkv, d, scale):
    """Per-sequence PyTorch evaluation (CPU oracle path)."""
    outs = []
    rep = hq // hkv
    for b in range(len(meta.cu_q_host) - 1):
        q0, q1 = meta.cu_q_host[b], meta.cu_q_host[b + 1]
        k0, k1 = meta.k_ranges[b]
        lq, lk = q1 - q0, k1 - k0
        qb = q[q0:q1].reshape(lq, hq, d).float()
        kb = k[k0:k1].reshape(lk, hkv, d).float()
        vb = v[k0:k1].reshape(lk, hkv, d).float()
        if rep > 1:
            kb = kb.repeat_interleave(rep, dim=1)
            vb = vb.repeat_interleave(rep, dim=1)
        s_ = torch.einsum("qhd,khd->hqk", qb, kb) * scale
        if meta.causal:
            ii = torch.arange(lq, device=q.device).unsqueeze(1) + (lk - lq)
            jj = torch.arange(lk, device=q.device).unsqueeze(0)
            allow = jj <= ii
            if meta.bidir_q is not None and meta.bidir_k is not None:
                allow = allow | (meta.bidir_q[q0:q1].bool().unsqueeze(1) & meta.bidir_k[k0:k1].bool().unsqueeze(0))
            s_ = s_.masked_fill(~allow.unsqueeze(0), float("-inf"))
        p = torch.softmax(s_, dim=-1)
        outs.append(torch.einsum("hqk,khd->qhd", p, vb).reshape(lq, hq * d))
    return torch.cat(outs, dim=0).to(q.dtype)


def _attn_flags(meta: AttnMeta):
    has_bidir = meta.causal and meta.bidir_q is not None and meta.bidir_k is not None
    causal_self = meta.causal and meta.self_attn and not has_bidir
    return has_bidir, causal_self


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, meta, hq, hkv, d, scale):
        qtab, ktab = meta.device_tables(q.device)
        has_bidir, _ = _attn_flags(meta)
        out, lse = _C().attn_fwd(q, k, v, qtab, ktab, int(hq), int(hkv), int(d), float(scale), has_bidir)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.meta, ctx.hq, ctx.hkv, ctx.d, ctx.scale = meta, hq, hkv, d, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        qtab, ktab = ctx.meta.device_tables(q.device)
        has_bidir, causal_self = _attn_flags(ctx.meta)
        dq = torch.empty((q.shape[0], q.shape[1]), device=q.device, dtype=q.dtype)
        dk = torch.empty((k.shape[0], k.shape[1]), device=q.device, dtype=q.dtype)
        dv = torch.empty((v.shape[0], v.shape[1]), device=q.device, dtype=q.dtype)
        _C().attn_bwd(dout.contiguous(), q, k, v, out, lse, qtab, ktab, dq, dk, dv, int(ctx.hq), int(ctx.hkv),
                      int(ctx.d), float(ctx.scale), has_bidir, causal_self)
        return dq, dk, dv, None, None, None, None, None


class _AttnPackedFn(torch.autograd.Function):
    """Self-attention on one packed q|k|v buffer; the three gradients are written straight into
    the column ranges of one ``dqkv`` buffer (no slice-backward copies)."""

    @staticmethod
    def forward(ctx, qkv, meta, hq, hkv, d, scale):
        qtab, ktab = meta.device_tables(qkv.device)
        has_bidir, _ = _attn_flags(meta)
        q, k, v = qkv[:, : hq * d], qkv[:, hq * d:(hq + hkv) * d], qkv[:, (hq + hkv) * d:]
        out, lse = _C().attn_fwd(q, k, v, qtab, ktab, int(hq), int(hkv), int(d), float(scale), has_bidir)
        ctx.save_for_backward(qkv, out, lse)
        ctx.meta, ctx.hq, ctx.hkv, ctx.d, ctx.scale = meta, hq, hkv, d, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        hq, hkv, d = ctx.hq, ctx.hkv, ctx.d
        qtab, ktab = ctx.meta.device_tables(qkv.device)
        has_bidir, causal_self = _attn_flags(ctx.meta)
        dqkv = torch.empty_like(qkv)
        q, k, v = qkv[:, : hq * d], qkv[:, hq * d:(hq + hkv) * d], qkv[:, (hq + hkv) * d:]
        dq, dk, dv = dqkv[:, : hq * d], dqkv[:, hq * d:(hq + hkv) * d], dqkv[:, (hq + hkv) * d:]
        _C().attn_bwd(dout.contiguous(), q, k, v, out, lse, qtab, ktab, dq, dk, dv, int(hq), int(hkv), int(d),
                      float(ctx.scale), has_bidir, causal_self)
        return dqkv, None, None, None, None, None


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, meta: AttnMeta, hq: int, hkv: int, d: int,
              scale: Optional[float] = None) -> torch.Tensor:
    """Varlen attention. ``q [Tq, hq*d]``, ``k/v [Tk, hkv*d]`` (row-strided views are fine);
    returns ``[Tq, hq*d]``. See :class:`AttnMeta` for the masking rule.

    Replaces flash-attn's ``flash_attn_func`` / ``flash_attn_varlen_func``
    (modeling_qwen2_5_vl.py:208-210, 1008-1015) and, with a key range longer than the query range,
    the reference's full-sequence recompute per denoise step (modeling_qwen2_5_vl_act.py:1906-1952)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if _is_cuda(q):
        return _AttnFn.apply(q, k, v, meta, hq, hkv, d, scale)
    return _attention_torch(q, k, v, meta, hq, hkv, d, scale)


DECODE_MAX_ROWS = 128  # query rows up to which the cached step uses the small-query attention kernel


def cached_step_kernels_usable(qkv: torch.Tensor, d: int) -> bool:
    """True when the fused rotary + cache write and the small-query attention kernel can serve this call: CUDA,
    inference (they have no backward), contiguous bf16 q|k|v."""
    return (_is_cuda(qkv) and not torch.is_grad_enabled() and qkv.dtype == torch.bfloat16 and qkv.is_contiguous()
            and d % 16 == 0)


def rope_cache_(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, cache_rows: torch.Tensor, cache: torch.Tensor,
                hq: int, hkv: int, d: int) -> torch.Tensor:
    """Rotary on the q and k heads of ``qkv`` (q rotated in place) with the rotated k and the v columns of row ``t``
    written to row ``cache_rows[t]`` of ``cache [rows, 2 * hkv * d]``: the rotary kernel and the index copy of the
    cached step in one launch. Returns ``qkv`` (only its q columns are meaningful afterwards)."""
    _C().rope_cache(qkv, cos, sin, cache_rows, cache, int(hq), int(hkv), int(d))
    return qkv


def attention_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, meta: AttnMeta, hq: int, hkv: int, d: int,
                     scale: Optional[float] = None) -> torch.Tensor:
    """:func:`attention` for a handful of query rows over a long cached key range (decode and denoise steps): one CTA
    per query row and key-value head with the keys staged in shared memory (csrc/decode.cu). Inference only; falls
    back to :func:`attention` for shapes the kernel does not serve."""
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if not (_is_cuda(q) and not torch.is_grad_enabled() and q.shape[0] <= DECODE_MAX_ROWS
            and _C().attn_decode_supported(q.shape[0], hq, hkv, d)):
        return attention(q, k, v, meta, hq, hkv, d, scale)
    qtab, ktab = meta.device_tables(q.device)
    max_keys = max((k1 - k0 for k0, k1 in meta.k_ranges), default=0)
    return _C().attn_decode(q, k, v, qtab, ktab, int(hq), int(hkv), int(d), float(scale), int(max_keys))


def attention_packed(qkv: torch.Tensor, meta: AttnMeta, hq: int, hkv: int, d: int,
                     scale: Optional[float] = None) -> torch.Tensor:
    """Self-attention over a packed ``[T, (hq + 2 hkv) * d]`` q|k|v buffer -> ``[T, hq * d]``."""
    if _is_cuda(qkv):
        scale = scale if scale is not None else 1.0 / math.sqrt(d)
        return _AttnPackedFn.apply(qkv.contiguous(), meta, hq, hkv, d, scale)
    q = qkv[:, : hq * d]
    k = qkv[:, hq * d:(hq + hkv) * d]
    v = qkv[:, (hq + hkv) * d:]
    return attention(q, k, v, meta, hq, hkv, d, scale)


# ----------------------------------------------------------------------------- fused LM head + CE
class _LmHeadCeFn(torch.autograd.Function):
    """Chunked LM head + cross entropy: logits exist only one vocabulary-wide row block at a time
    and only for rows that carry a label."""

    CHUNK = 4096

    @staticmethod
    def _logits_buffer(rows: int, V: int, device) -> torch.Tensor:
        # the backward pass reads the logits as a GEMM operand through TMA: the row pitch must be a
        # multiple of 16 bytes even when the vocabulary size is not a multiple of 8
        Vp = (V + 7) // 8 * 8
        return torch.empty((rows, Vp), device=device, dtype=torch.bfloat16)[:, :V]

    @staticmethod
    def forward(ctx, hidden, weight, labels):
        R = hidden.shape[0]
        V = weight.shape[0]
        loss = torch.empty(R, device=hidden.device, dtype=torch.float32)
        pred = torch.empty(R, device=hidden.device, dtype=torch.int64)
        lse = torch.empty(R, device=hidden.device, dtype=torch.float32)
        w2 = _aligned2d(weight)
        for s in range(0, R, _LmHeadCeFn.CHUNK):
            e = min(R, s + _LmHeadCeFn.CHUNK)
            logits = _LmHeadCeFn._logits_buffer(e - s, V, hidden.device)
            G.launch([G.GemmSpec(hidden[s:e], w2, logits)])
            _C().ce_fwd(logits, labels[s:e], loss[s:e], lse[s:e], pred[s:e])
        ctx.save_for_backward(hidden, weight, labels, lse)
        ctx.mark_non_differentiable(pred)
        return loss, pred

    @staticmethod
    def backward(ctx, dloss, _dpred):
        hidden, weight, labels, lse = ctx.saved_tensors
        R, V = hidden.shape[0], weight.shape[0]
        w2 = _aligned2d(weight)
        dh = torch.empty_like(hidden)
        dw = torch.zeros((V, hidden.shape[1]), device=hidden.device, dtype=torch.float32)
        dloss = dloss.contiguous().float()
        for s in range(0, R, _LmHeadCeFn.CHUNK):
            e = min(R, s + _LmHeadCeFn.CHUNK)
            logits = _LmHeadCeFn._logits_buffer(e - s, V, hidden.device)
            G.launch([G.GemmSpec(hidden[s:e], w2, logits)])
            _C().ce_bwd(logits, labels[s:e], lse[s:e], dloss[s:e])  # in place: logits -> dlogits
            G.launch([G.GemmSpec(logits, w2, dh[s:e], b_mn=True)])
            G.launch([G.GemmSpec(logits, hidden[s:e], dw, a_mn=True, b_mn=True, flags=G.OUT_FP32 | G.ACCUMULATE)])
        return dh, dw.to(weight.dtype), None


def lm_head_ce(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor):
    """Per-row cross entropy (0 where ``labels == -100``) and arg-max ids for ``[R, H]`` rows.

    The reference materialises ``[B, S, V]`` logits for every position and then computes an
    unreduced CE (modeling_qwen2_5_vl_act.py:1406-1444); here only labelled rows reach the head
    and logits live one row block at a time."""
    if _is_cuda(hidden):
        return _LmHeadCeFn.apply(hidden.contiguous(), weight, labels.contiguous())
    return ref.lm_head_ce(hidden, weight, labels)


# ----------------------------------------------------------------------------- misc gathers
class _GatherRowsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx, out_rows):
        ctx.save_for_backward(idx)
        ctx.in_rows = x.shape[0]
        return x.index_select(0, idx)

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        dx = dy.new_zeros((ctx.in_rows, dy.shape[1]))
        dx.index_add_(0, idx, dy)
        return dx, None, None


def gather_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    return x.index_select(0, idx)


# ----------------------------------------------------------------------------- optional NVTX ranges
NVTX_OPS = ("linear", "linear_gelu", "rms_norm", "swiglu_ffn", "gate_up_swiglu", "moe_ffn", "rope_qk", "attention",
            "attention_packed", "lm_head_ce", "column_sum", "make_route_plan")


def _annotate():
    import sys

    from ..utils import nvtx

    return nvtx.annotate_module(sys.modules[__name__], NVTX_OPS)


_annotate()

"""Whole transformer blocks as one autograd node backed by one host call per direction.

The decoder layer and the vision block are the same pre-norm pattern (RMSNorm -> fused QKV -> rotary -> varlen
attention -> output projection + residual -> RMSNorm -> SwiGLU FFN + residual, the FFN being dense or the token-type
routed dual-expert one). :func:`transformer_block` runs that pattern through ``csrc/blocks.cpp``: the same kernels
as the operator-by-operator path of :mod:`wallx_b200.ops.functional`, enqueued by a single C++ call for the forward
and one for the backward, so the host spends microseconds instead of milliseconds per layer and results are
bit-identical. Row-sharded weights (``parallel/zero3.py``) are gathered inside the GEMMs exactly as in the Python
path; weight gradients go straight into their sinks.

Reference: ``Qwen2_5_VLDecoderLayer_with_MoE`` (modeling_qwen2_5_vl_act.py:172-273) and ``Qwen2_5_VLVisionBlock``
(modeling_qwen2_5_vl.py:365-391), which run as 20-30 separate framework calls each way.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import torch

from . import _ext
from . import functional as F_

ENABLED = os.environ.get("WALLX_FUSED_BLOCKS", "1") != "0"
PREFETCH_NEXT = os.environ.get("WX_AG_PREFETCH_NEXT", "1") != "0"


_PULLERS = None


def _default_pullers() -> int:
    global _PULLERS
    if _PULLERS is None:
        from ..parallel.ag_linear import DEFAULT_PULLERS

        _PULLERS = DEFAULT_PULLERS
    return _PULLERS


def _wtuple(w: torch.Tensor, sink, forward: bool, gather: bool = True):
    """(weight or staging view, sink view or None, peers, flags, rows per rank, rank, copy CTAs, epoch).
    ``gather=False``: the weight is already whole in its staging view, no gather is enqueued for it by this call."""
    gw = F_._shard_of(w)
    sview = sink[0] if sink is not None else None
    if gw is None:
        return (w, sview, [], None, 0, 0, 0, 0)
    gw.pin_pullers(gw.n_pullers or _default_pullers())
    return (w, sview, gw.peer_ptrs, gw.flags, gw.rows_per_rank, gw.rank, gw.n_pullers,
            gw.next_epoch() if gather else max(gw.epoch, 1))


# The down-projection weights of the block whose forward ran last: its backward runs right after the backward of
# the block that is running forward now, so that block's backward gathers them ahead of time (row-sharded weights).
_PREV_DOWN = []


class _BlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ln1_w, w_qkv, b_qkv, w_o, b_o, ln2_w, b_gu, b_dn, cfg, *ffn_w):
        C = _ext.get()
        meta, cos, sin, n_rot, hq, hkv, d, scale, eps, plan = cfg
        qtab, ktab = meta.device_tables(x.device)
        has_bidir, causal_self = F_._attn_flags(meta)
        need_bwd = any(ctx.needs_input_grad)
        weights = [w_qkv, w_o, *ffn_w]
        sinks = [F_._sink_of(w) if need_bwd else None for w in weights]
        wt = [_wtuple(w, None, True) for w in weights]
        moe = plan is not None
        res = C.block_fwd(x, ln1_w, wt[0], b_qkv, cos, sin, int(n_rot), qtab, ktab, int(hq), int(hkv), int(d), float(scale),
                          bool(has_bidir), wt[1], b_o, ln2_w, float(eps), wt[2:], b_gu, b_dn,
                          plan.dest if moe else None, plan.seg if moe else None, plan.inv if moe else None,
                          int(plan.rows) if moe else 0, bool(need_bwd))
        out = res[0]
        global _PREV_DOWN
        prev_down, _PREV_DOWN = _PREV_DOWN, [ffn_w[2 * e + 1] for e in range(len(ffn_w) // 2)]
        if need_bwd:
            ctx.prev_down = [w for w in prev_down if F_._shard_of(w) is not None][:2]
            y1, rstd1, qkv, o_attn, lse, x2, rstd2, xn, gu, h = res[1:]
            ctx.save_for_backward(x, ln1_w, y1, rstd1, qkv, o_attn, lse, x2, ln2_w, rstd2, xn, gu, h, cos, sin, qtab, ktab,
                                  w_qkv, w_o, *ffn_w)
            ctx.cfg = (int(n_rot), int(hq), int(hkv), int(d), float(scale), bool(has_bidir), bool(causal_self), plan)
            ctx.has_bias = (b_qkv is not None, b_o is not None, b_gu is not None, b_dn is not None)
            ctx.sinks = sinks
        return out

    @staticmethod
    def backward(ctx, dout):
        C = _ext.get()
        (x, ln1_w, y1, rstd1, qkv, o_attn, lse, x2, ln2_w, rstd2, xn, gu, h, cos, sin, qtab, ktab, w_qkv, w_o,
         *ffn_w) = ctx.saved_tensors
        n_rot, hq, hkv, d, scale, has_bidir, causal_self, plan = ctx.cfg
        weights = [w_qkv, w_o, *ffn_w]
        sinks = ctx.sinks
        n_exp = len(ffn_w) // 2
        downs = [ffn_w[2 * e + 1] for e in range(n_exp)]
        dn_shards = [F_._shard_of(w) for w in downs]
        # the block whose backward ran just before this one may have gathered this block's down projections already
        dn_in_place = bool(dn_shards) and all(g is not None and g.in_place() for g in dn_shards)
        wt = [_wtuple(w, s, False, gather=not (dn_in_place and any(w is d_ for d_ in downs)))
              for w, s in zip(weights, sinks)]
        for g in dn_shards:
            if g is not None:
                g.prefetched = False  # consumed by this backward
        # gathers of the next block's down projections ride on this block's last weight-gradient launch; after it the
        # two staging slots belong to them
        nxt = ctx.prev_down if PREFETCH_NEXT and all(F_._shard_of(w) is not None for w in weights) else []
        if len({F_._shard_of(w).slot for w in nxt}) != len(nxt):
            nxt = []
        moe = plan is not None
        hb = ctx.has_bias
        res = C.block_bwd(dout, x, ln1_w, y1, rstd1, qkv, o_attn, lse, x2, ln2_w, rstd2, xn, gu, h, wt[0], hb[0], cos, sin,
                          n_rot, qtab, ktab, hq, hkv, d, scale, has_bidir, causal_self, wt[1], hb[1], wt[2:], hb[2], hb[3],
                          plan.dest if moe else None, plan.seg if moe else None, plan.segk if moe else None,
                          int(plan.rows) if moe else 0, dn_in_place, [_wtuple(w, None, False) for w in nxt])
        for w in nxt:
            F_._shard_of(w).prefetched = True
        dx, dln1, dln2, db_qkv, db_o, db_gu, db_dn, dw_qkv, dw_o = res[:9]
        dw_ffn = list(res[9:])
        # sink callbacks in the order the gradients were produced (all of them are enqueued by now)
        order = []
        order += [2 + 2 * e + 1 for e in range(n_exp)] + [2 + 2 * e for e in range(n_exp)] + [1, 0]
        for i in order:
            if sinks[i] is not None:
                sinks[i][1]()
        return (dx, dln1, dw_qkv, db_qkv, dw_o, db_o, dln2, db_gu, db_dn, None, *dw_ffn)


def usable(x: torch.Tensor) -> bool:
    return ENABLED and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2


def transformer_block(x: torch.Tensor, ln1_w, w_qkv, b_qkv, w_o, b_o, ln2_w, ffn_w: Sequence[torch.Tensor], b_gu, b_dn, *,
                      meta: F_.AttnMeta, cos, sin, n_rot: int, hq: int, hkv: int, d: int, eps: float,
                      plan: Optional[F_.RoutePlan] = None, scale: Optional[float] = None) -> torch.Tensor:
    """``x + attn(norm1(x))`` then ``. + ffn(norm2(.))`` on packed rows ``[T, C]``.

    ``ffn_w`` is ``(gate_up, down)`` for a dense SwiGLU FFN or ``(gate_up_0, down_0, gate_up_1, down_1, ...)`` with a
    routing ``plan`` for the token-type routed experts. Self-attention over the packed q|k|v buffer with ``meta``."""
    import math

    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    cfg = (meta, cos, sin, n_rot, hq, hkv, d, scale, eps, plan)
    return _BlockFn.apply(x.contiguous(), ln1_w, w_qkv, b_qkv, w_o, b_o, ln2_w, b_gu, b_dn, cfg, *ffn_w)

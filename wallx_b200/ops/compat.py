"""Operator-level API with the reference's names and signatures (wall_x/fusions/ops.py), for code
written against ``wall_x.fusions.ops``. Each function runs this framework's kernels on CUDA
tensors and the PyTorch oracle on CPU tensors, and is differentiable.

* ``asym_dual_gmm(in0, in1, w0, w1, trans_b)``: two independent GEMMs in one launch (:6-165)
* ``permute(x, indices)`` / ``unpermute(x, row_id_map, probs)``: stable grouping by expert id and
  its inverse (:175-392); compact layout (no padding rows), ``row_id_map[t]`` = grouped row of token t
* ``multimodal_rope(q, k, cos, sin, mrope_section)``: ``[B, H, S, D]`` layout, ``cos/sin [3, B, S, D]``,
  the contiguous section layout of the reference CUDA kernel (:402-497)
* ``get_rope_index`` / ``rot_pos_emb`` / ``get_window_index`` (:507-742)
"""
from __future__ import annotations

from typing import Sequence

import torch

from . import backend as BE
from . import functional as F_
from . import gemm as G
from . import index as IX
from . import ref
from .index import get_rope_index  # noqa: F401


class AsymmetricDualExpertGemm(torch.autograd.Function):
    """``apply(in0, in1, w0, w1, trans_b)``: forward, dgrad and wgrad are one two-problem launch each (ops.py:6-165)."""

    @staticmethod
    def forward(ctx, a0, a1, w0, w1, trans_b):
        ctx.save_for_backward(a0, a1, w0, w1)
        ctx.trans_b = trans_b
        n0 = w0.shape[0] if trans_b else w0.shape[1]
        n1 = w1.shape[0] if trans_b else w1.shape[1]
        o0 = torch.empty((a0.shape[0], n0), device=a0.device, dtype=a0.dtype)
        o1 = torch.empty((a1.shape[0], n1), device=a1.device, dtype=a1.dtype)
        specs = [G.GemmSpec(a, w, o, b_mn=not trans_b) for a, w, o in ((a0, w0, o0), (a1, w1, o1)) if a.shape[0] > 0]
        if specs:
            G.launch(specs)
        return o0, o1

    @staticmethod
    def backward(ctx, g0, g1):
        a0, a1, w0, w1 = ctx.saved_tensors
        tb = ctx.trans_b
        g0, g1 = g0.contiguous(), g1.contiguous()
        da0, da1 = torch.zeros_like(a0), torch.zeros_like(a1)
        dw0, dw1 = torch.zeros_like(w0), torch.zeros_like(w1)
        # dgrad: dA = dY W (trans_b) or dY W^T
        specs = [G.GemmSpec(g, w, d, b_mn=tb) for g, w, d in ((g0, w0, da0), (g1, w1, da1)) if g.shape[0] > 0]
        if specs:
            G.launch(specs)
        # wgrad: dW[n, k] = dY^T A (trans_b) or dW[k, n] = A^T dY
        specs = []
        for g, a, d in ((g0, a0, dw0), (g1, a1, dw1)):
            if g.shape[0] == 0:
                continue
            specs.append(G.GemmSpec(g, a, d, a_mn=True, b_mn=True) if tb else G.GemmSpec(a, g, d, a_mn=True, b_mn=True))
        if specs:
            G.launch(specs)
        return da0, da1, dw0, dw1, None


def asym_dual_gmm(input_expert0, input_expert1, weight_expert0, weight_expert1, trans_b: bool = False):
    if input_expert0.is_cuda:
        mk = lambda t: F_._aligned2d(t.contiguous())
        return AsymmetricDualExpertGemm.apply(mk(input_expert0), mk(input_expert1), mk(weight_expert0), mk(weight_expert1), trans_b)
    f = (lambda a, w: a @ w.t()) if trans_b else (lambda a, w: a @ w)
    return f(input_expert0, weight_expert0), f(input_expert1, weight_expert1)


class PermuteMoE_topK(torch.autograd.Function):
    """``apply(input_act, indices, num_out_tokens, max_token_num) -> (permuted, row_id_map)``.

    ``indices`` is ``[T]`` (top-1, the token-type routing of this model) or ``[T, K]``; rows are grouped
    by a stable sort of the flattened expert ids; ``row_id_map[k * T + t]`` (int32) is the row of token
    t's k-th copy. The backward pass sums the gradients of a token's copies (ops.py:175-274).
    """

    @staticmethod
    def forward(ctx, input_act, indices, num_out_tokens=0, max_token_num=0):
        if not input_act.numel():
            return input_act, None
        out, row_id_map = BE.permute(input_act, indices, int(num_out_tokens or 0), None, int(max_token_num or 0))
        ctx.row_id_map = row_id_map
        ctx.topk = 1 if indices.dim() == 1 else int(indices.shape[1])
        ctx.mark_non_differentiable(row_id_map)
        return out, row_id_map

    @staticmethod
    def backward(ctx, g, _):
        if not g.numel():
            return g, None, None, None
        return BE.unpermute(g.contiguous(), ctx.row_id_map, None, 0, ctx.topk), None, None, None


class UnpermuteMoE_topK(torch.autograd.Function):
    """``apply(input_act, row_id_map, probs=None) -> [T, C]``: the inverse gather, with the K copies of a
    token weighted by ``probs [T, K]`` and summed; differentiable in the rows and in ``probs`` (ops.py:284-383)."""

    @staticmethod
    def forward(ctx, input_act, row_id_map, probs=None):
        if not input_act.numel():
            ctx.probs = probs
            return input_act
        ctx.save_for_backward(input_act, row_id_map)
        ctx.probs = probs
        return BE.unpermute(input_act, row_id_map, probs, 0, 1 if probs is None else int(probs.reshape(-1, probs.shape[-1]).shape[1]))

    @staticmethod
    def backward(ctx, g):
        if not g.numel():
            return g, None, None
        x, row_id_map = ctx.saved_tensors
        probs = ctx.probs
        if probs is None and row_id_map.numel() != g.shape[0]:  # top-K copies without weights
            k = row_id_map.numel() // g.shape[0]
            probs = torch.ones((g.shape[0], k), device=g.device, dtype=g.dtype)
            dx, _ = BE.unpermute_bwd(g.contiguous(), x, row_id_map, probs)
            return dx, None, None
        dx, dp = BE.unpermute_bwd(g.contiguous(), x, row_id_map, probs)
        return dx, None, (dp if probs is not None and probs.requires_grad else None)


def permute(input_act, indices, num_out_tokens=None, max_token_num=0):
    """Returns ``(permuted_act, row_id_map)`` with ``row_id_map`` int32 ``[K * T]``."""
    return PermuteMoE_topK.apply(input_act, indices, 0 if num_out_tokens is None else num_out_tokens, max_token_num)


def unpermute(input_act, row_id_map, probs=None):
    return UnpermuteMoE_topK.apply(input_act, row_id_map, probs)


class MultimodalRoPE(torch.autograd.Function):
    """``apply(q, k, cos, sin, mrope_section) -> (q_out, k_out)`` in the reference's ``[B, H, S, D]`` layout with
    its contiguous channel-to-axis rule; fresh outputs, backward = the transposed rotation (ops.py:402-497)."""

    @staticmethod
    def forward(ctx, q, k, cos, sin, mrope_section):
        if len(mrope_section) != 3:
            raise RuntimeError("mrope_section must hold three integers (frequency pairs for t, h, w)")
        doubled = [2 * int(x) for x in mrope_section]
        q_out, k_out = torch.empty_like(q), torch.empty_like(k)
        BE.rope(q, k, cos, sin, q_out, k_out, doubled)
        ctx.save_for_backward(cos, sin)
        ctx.doubled = doubled
        return q_out, k_out

    @staticmethod
    def backward(ctx, gq, gk):
        cos, sin = ctx.saved_tensors
        dq, dk = torch.empty_like(gq), torch.empty_like(gk)
        BE.rope_bwd(gq, gk, None, None, cos, sin, dq, dk, ctx.doubled)
        return dq, dk, None, None, None


def multimodal_rope(q, k, cos, sin, mrope_section: Sequence[int]):
    """q ``[B, Hq, S, D]``, k ``[B, Hkv, S, D]``, cos/sin ``[3, B, S, D]`` -> rotated (q, k)."""
    B, Hq, S, D = q.shape
    Hk = k.shape[1]
    ax = ref.mrope_axis_of_channel(D, list(mrope_section), "wallx_cuda").to(q.device)
    sel = ax.view(1, 1, 1, D).expand(1, B, S, D)
    c = cos.float().gather(0, sel).squeeze(0).reshape(B * S, D).contiguous()
    s = sin.float().gather(0, sel).squeeze(0).reshape(B * S, D).contiguous()
    packed = torch.cat([q.permute(0, 2, 1, 3).reshape(B * S, Hq * D), k.permute(0, 2, 1, 3).reshape(B * S, Hk * D)], dim=1)
    out = F_.rope_qk(packed, c, s, Hq + Hk, D)
    qo = out[:, : Hq * D].reshape(B, S, Hq, D).permute(0, 2, 1, 3)
    ko = out[:, Hq * D:].reshape(B, S, Hk, D).permute(0, 2, 1, 3)
    return qo, ko


def rot_pos_emb(inv_freq, grid_thw, spatial_merge_size: int):
    return IX.rot_pos_emb(inv_freq, grid_thw, spatial_merge_size)


def get_window_index(grid_thw, window_size: int, spatial_merge_size: int, patch_size: int, spatial_merge_unit: int = 4):
    return IX.get_window_index(grid_thw, window_size, spatial_merge_size, patch_size, spatial_merge_unit)

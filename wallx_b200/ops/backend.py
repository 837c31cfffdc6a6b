"""Low-level operator entry points with the reference's backend signatures (wall_x/fusions/backend.py).

The reference keeps one thin Python function per pybind symbol: the caller passes pre-allocated
outputs and workspaces and the function forwards them to the CUDA extension. Code written against
that layer (``from wall_x.fusions import backend``) finds the same names here:

* ``asym_dual_gmm_separated`` (backend.py:71-135): two independent GEMMs, optional caller outputs
* ``permute`` / ``unpermute`` / ``unpermute_bwd`` (backend.py:138-230): top-K token grouping
* ``rope`` / ``rope_bwd`` (backend.py:233-299): 3-axis rotary on ``[B, H, S, D]`` into caller buffers
* ``get_rope_index`` / ``rot_pos_emb`` / ``get_window_index`` (backend.py:302-433)

None of these is differentiable (the autograd layer is ``wallx_b200.ops.compat``). CUDA tensors
run this framework's kernels where one exists for the layout (GEMMs, rotary, index generation);
top-1 grouping of bf16 rows uses the row-copy kernels (``permute_rows`` / ``gather_rows``), top-K with
probabilities uses index operations: the model itself never materialises a permutation, it fuses the
routing into the RMSNorm store and the down-projection epilogue.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from . import index as IX
from . import ref


# ----------------------------------------------------------------------------- grouped GEMM
def asym_dual_gmm_separated(input_expert0: torch.Tensor, input_expert1: torch.Tensor, weight_expert0: torch.Tensor,
                            weight_expert1: torch.Tensor, output_expert0: Optional[torch.Tensor] = None,
                            output_expert1: Optional[torch.Tensor] = None, trans_a: bool = False,
                            trans_b: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``out_e = op(input_e) @ op(weight_e)`` for both experts in one launch.

    ``trans_a``: inputs are stored ``[k, m]``; ``trans_b``: weights are stored ``[n, k]``.
    """
    outs = []
    for a, w, o in ((input_expert0, weight_expert0, output_expert0), (input_expert1, weight_expert1, output_expert1)):
        m = a.shape[1] if trans_a else a.shape[0]
        n = w.shape[0] if trans_b else w.shape[1]
        if o is None:
            o = torch.empty((m, n), device=a.device, dtype=a.dtype)
        elif tuple(o.shape) != (m, n):
            raise ValueError(f"output has shape {tuple(o.shape)}, the product has {(m, n)}")
        outs.append(o)
    if input_expert0.is_cuda:
        from . import functional as F_
        from . import gemm as G

        # the core computes D[M, N] = A[M, K] * B[N, K]^T; ``a_mn`` / ``b_mn`` mark operands stored with the
        # contraction dimension outermost, which is trans_a / not trans_b here
        specs, copies = [], []
        for a, w, o in ((input_expert0, weight_expert0, outs[0]), (input_expert1, weight_expert1, outs[1])):
            if o.numel() == 0:
                continue
            dst = o if F_._pitch_ok(o) else F_._aligned2d(torch.empty_like(o))
            if dst is not o:
                copies.append((o, dst))
            specs.append(G.GemmSpec(F_._aligned2d(a.contiguous()), F_._aligned2d(w.contiguous()), dst, a_mn=trans_a,
                                    b_mn=not trans_b))
        if specs:
            G.launch(specs)
        for o, dst in copies:
            o.copy_(dst)
    else:
        for a, w, o in ((input_expert0, weight_expert0, outs[0]), (input_expert1, weight_expert1, outs[1])):
            aa = a.t() if trans_a else a
            ww = w.t() if trans_b else w
            o.copy_((aa.float() @ ww.float()).to(o.dtype))
    return outs[0], outs[1]


# ----------------------------------------------------------------------------- top-K grouping
def _row_kernels_apply(x: torch.Tensor) -> bool:
    """The row-copy kernels move bf16 rows in 16-byte pieces."""
    return x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] % 8 == 0 and x.shape[0] > 0


def sorted_rows(indices: torch.Tensor) -> torch.Tensor:
    """Row of every (token, k) pair after a stable sort of the flattened expert ids: ``[T, K]`` long."""
    idx = indices.reshape(indices.shape[0], -1)
    flat = idx.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices
    pos = torch.empty_like(order)
    pos[order] = torch.arange(order.numel(), device=flat.device)
    return pos.view(idx.shape)


def permute(input: torch.Tensor, indices: torch.Tensor, num_out_tokens: int = 0, workspace: Optional[torch.Tensor] = None,
            max_expanded_token_num: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Group token rows by expert id. ``indices`` is ``[T]`` or ``[T, K]``.

    Returns ``(permuted [rows, C], row_id_map int32 [K * T])`` with ``row_id_map[k * T + t]`` the row
    of token t's k-th copy; ``rows = num_out_tokens`` when positive (later rows are dropped), else
    ``T * K``. ``workspace`` and ``max_expanded_token_num`` exist for signature parity: nothing here
    needs a sort workspace.
    """
    pos = sorted_rows(indices)  # [T, K]
    T, K = pos.shape
    rows = int(num_out_tokens) if num_out_tokens and num_out_tokens > 0 else T * K
    if _row_kernels_apply(input) and K == 1 and rows == T:  # the top-1 routing of this model: one row-copy kernel
        from . import _ext

        dest = pos.reshape(-1).to(torch.int32)
        return _ext.get().permute_rows(input.contiguous(), dest, rows), dest
    out = input.new_zeros((rows, input.shape[1]))
    src = torch.arange(T, device=input.device).view(T, 1).expand(T, K).reshape(-1)
    flat = pos.reshape(-1)
    keep = flat < rows
    out.index_copy_(0, flat[keep], input.index_select(0, src[keep]))
    return out, pos.t().reshape(-1).to(torch.int32)


def _acc_dtype(t: torch.Tensor) -> torch.dtype:
    return torch.promote_types(t.dtype, torch.float32)


def unpermute(input: torch.Tensor, row_id_map: torch.Tensor, prob: Optional[torch.Tensor] = None, max_tokens: int = 0,
              num_topK: int = 1) -> torch.Tensor:
    """``out[t] = sum_k prob[t, k] * input[row_id_map[k * T + t]]`` (rows beyond ``input`` count as dropped)."""
    K = int(prob.shape[1]) if prob is not None and prob.dim() == 2 else max(int(num_topK), 1)
    T = row_id_map.numel() // K
    if prob is None and K == 1 and input.shape[0] == T and _row_kernels_apply(input) and row_id_map.dtype == torch.int32:
        from . import _ext

        return _ext.get().gather_rows(input.contiguous(), row_id_map.contiguous())  # nothing was dropped: a plain gather
    acc = _acc_dtype(input)
    rows = row_id_map.view(K, T).long()
    valid = rows < input.shape[0]
    g = input.index_select(0, rows.clamp(max=max(input.shape[0] - 1, 0)).reshape(-1)).view(K, T, -1).to(acc)
    g = g * valid.unsqueeze(-1)
    if prob is not None:
        g = g * prob.reshape(T, K).t().unsqueeze(-1).to(acc)
    return g.sum(0).to(input.dtype)


def unpermute_bwd(input_bwd: torch.Tensor, input_fwd: torch.Tensor, row_id_map: torch.Tensor,
                  prob: Optional[torch.Tensor]) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Gradients of :func:`unpermute`: ``(d input_fwd [rows, C], d prob [T, K] or None)``."""
    K = int(prob.shape[1]) if prob is not None and prob.dim() == 2 else 1
    T = row_id_map.numel() // K
    acc = _acc_dtype(input_fwd)
    rows = row_id_map.view(K, T).long()
    valid = rows < input_fwd.shape[0]
    safe = rows.clamp(max=max(input_fwd.shape[0] - 1, 0))
    g = input_bwd.to(acc).unsqueeze(0).expand(K, T, -1)  # gradient reaching every copy
    scale = valid.unsqueeze(-1).to(acc)
    if prob is not None:
        scale = scale * prob.reshape(T, K).t().unsqueeze(-1).to(acc)
    d_in = torch.zeros(input_fwd.shape, dtype=acc, device=input_fwd.device)
    d_in.index_add_(0, safe.reshape(-1), (g * scale).reshape(K * T, -1))
    d_prob = None
    if prob is not None:
        fwd = input_fwd.index_select(0, safe.reshape(-1)).view(K, T, -1).to(acc)
        d_prob = ((fwd * g).sum(-1) * valid).t().contiguous().to(prob.dtype).view(prob.shape)
    return d_in.to(input_fwd.dtype), d_prob


# ----------------------------------------------------------------------------- rotary
def _rope_tables(cos: torch.Tensor, sin: torch.Tensor, D: int, doubled: Sequence[int]):
    """``[3, B, S, D]`` tables -> per-token ``[B * S, D]``: channel d takes its angle from axis t for
    ``d < doubled[0]``, h for the next ``doubled[1]`` channels, w for the rest (the reference kernel's rule)."""
    _, B, S, _ = cos.shape
    if len(doubled) != 3 or sum(int(x) for x in doubled) != D:
        raise ValueError(f"mrope_section_doubled {list(doubled)} must be three channel counts that add up to {D}")
    ax = ref.mrope_axis_of_channel(D, [int(x) // 2 for x in doubled], "wallx_cuda").to(cos.device)
    sel = ax.view(1, 1, 1, D).expand(1, B, S, D)
    c = cos.float().gather(0, sel).squeeze(0).reshape(B * S, D).contiguous()
    s = sin.float().gather(0, sel).squeeze(0).reshape(B * S, D).contiguous()
    return c, s


def _rope_apply(q, k, cos, sin, q_out, k_out, doubled: Sequence[int], transpose: bool) -> None:
    """Rotation (or its transpose, which is the gradient) of q and k into caller buffers."""
    B, Hq, S, D = q.shape
    Hk = k.shape[1]
    c, s = _rope_tables(cos, sin, D, doubled)
    packed = torch.cat([q.permute(0, 2, 1, 3).reshape(B * S, Hq * D), k.permute(0, 2, 1, 3).reshape(B * S, Hk * D)],
                       dim=1).contiguous()
    if packed.is_cuda and packed.dtype == torch.bfloat16:
        from . import _ext

        out = _ext.get().rope_qk(packed, c, s, Hq + Hk, D, bool(transpose))
    else:
        x = packed.view(B * S, Hq + Hk, D).float()
        h = D // 2
        if not transpose:  # y = x * c + rotate_half(x) * s
            out = x * c.unsqueeze(1) + torch.cat((-x[..., h:], x[..., :h]), dim=-1) * s.unsqueeze(1)
        else:  # dx = g * c + rotate_half^T(g * s), rotate_half^T(v) = [v2, -v1]
            gs = x * s.unsqueeze(1)
            out = x * c.unsqueeze(1) + torch.cat((gs[..., h:], -gs[..., :h]), dim=-1)
        out = out.reshape(B * S, (Hq + Hk) * D)
    q_out.copy_(out[:, : Hq * D].reshape(B, S, Hq, D).permute(0, 2, 1, 3))
    k_out.copy_(out[:, Hq * D:].reshape(B, S, Hk, D).permute(0, 2, 1, 3))


def rope(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, q_out: torch.Tensor, k_out: torch.Tensor,
         mrope_section_doubled: Sequence[int]) -> None:
    """Rotate q ``[B, Hq, S, D]`` and k ``[B, Hkv, S, D]`` into ``q_out`` / ``k_out`` (``cos`` / ``sin`` ``[3, B, S, D]``).
    ``mrope_section_doubled`` is the channel count per axis, e.g. ``[32, 48, 48]`` for D = 128."""
    _rope_apply(q, k, cos, sin, q_out, k_out, mrope_section_doubled, False)


def rope_bwd(grad_q_out: torch.Tensor, grad_k_out: torch.Tensor, q: Optional[torch.Tensor], k: Optional[torch.Tensor],
             cos: torch.Tensor, sin: torch.Tensor, grad_q: torch.Tensor, grad_k: torch.Tensor,
             mrope_section_doubled: Sequence[int]) -> None:
    """Gradient w.r.t. q and k, written into ``grad_q`` / ``grad_k``: the transposed rotation of the
    incoming gradients (the rotation is linear, so ``q`` and ``k`` themselves are not needed)."""
    _rope_apply(grad_q_out, grad_k_out, cos, sin, grad_q, grad_k, mrope_section_doubled, True)


# ----------------------------------------------------------------------------- index generation
def get_rope_index(input_ids, image_grid_thw, video_grid_thw, second_per_grid_ts, attention_mask, spatial_merge_size: int,
                   image_token_id: int, video_token_id: int, vision_start_token_id: int, tokens_per_second: float):
    return IX.get_rope_index(input_ids, image_grid_thw, video_grid_thw, second_per_grid_ts, attention_mask, spatial_merge_size,
                             image_token_id, video_token_id, vision_start_token_id, tokens_per_second)


def rot_pos_emb(inv_freq: torch.Tensor, grid_thw: torch.Tensor, spatial_merge_size: int) -> torch.Tensor:
    return IX.rot_pos_emb(inv_freq, grid_thw, spatial_merge_size)


def get_window_index(grid_thw: torch.Tensor, spatial_merge_size: int, vit_merger_window_size: int, patch_size: int,
                     spatial_merge_unit: int):
    """Here ``vit_merger_window_size`` is already ``window_size // spatial_merge_size // patch_size``
    (the reference's wrapper computes it, ops.py:685-742)."""
    window = int(vit_merger_window_size) * int(spatial_merge_size) * int(patch_size)
    return IX.get_window_index(grid_thw, window, spatial_merge_size, patch_size, spatial_merge_unit)

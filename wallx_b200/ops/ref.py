"""Plain PyTorch restatement of every operator (the CPU execution path and the numerics oracle).

Everything here is differentiable through ordinary autograd and runs in whatever dtype it is given
(fp32 on CPU). The CUDA kernels are tested against these functions.

Reference behaviour restated (not imported):
* RMSNorm, fp32 statistics, weight multiply in model dtype   - modeling_qwen2_5_vl.py:122-139
* 3-axis mRoPE, HF channel layout                            - modeling_qwen2_5_vl.py:731-773
* 3-axis mRoPE, contiguous layout of the CUDA kernel         - csrc/rope.cu:104-122, fusions/ops.py:451
* rope_index (t/h/w position ids + deltas)                   - modeling_qwen2_5_vl_act.py:929-1149
* ViT rot_pos_emb / get_window_index                         - modeling_qwen2_5_vl.py:473-547
* token-type permute / unpermute                             - modeling_qwen2_5_vl_act.py:138-157
* attention mask with the bidirectional action-token block   - modeling_qwen2_5_vl_act.py:616-637
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------- norms / activations
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return weight * (xf * torch.rsqrt(var + eps)).to(x.dtype)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int = 16) -> torch.Tensor:
    """[I, ...] gate and up rows -> [2I, ...] in blocks of ``block`` gate rows then ``block`` up rows."""
    I = gate.shape[0]
    assert I % block == 0
    rest = gate.shape[1:]
    g = gate.reshape(I // block, 1, block, *rest)
    u = up.reshape(I // block, 1, block, *rest)
    return torch.cat([g, u], dim=1).reshape(2 * I, *rest)


def deinterleave_gate_up(gu: torch.Tensor, block: int = 16, dim: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`interleave_gate_up` along ``dim``."""
    gu = gu.movedim(dim, 0)
    two_i = gu.shape[0]
    rest = gu.shape[1:]
    v = gu.reshape(two_i // (2 * block), 2, block, *rest)
    g = v[:, 0].reshape(two_i // 2, *rest).movedim(0, dim)
    u = v[:, 1].reshape(two_i // 2, *rest).movedim(0, dim)
    return g, u


def swiglu_interleaved(gu: torch.Tensor, block: int = 16) -> torch.Tensor:
    """``silu(gate) * up`` for a last dimension laid out ``[16 gate | 16 up | 16 gate | ...]``."""
    g, u = deinterleave_gate_up(gu, block, dim=-1)
    return F.silu(g) * u


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    return F.linear(x, w, b)


# ----------------------------------------------------------------------------- rotary embeddings
def rope_inv_freq(head_dim: int, theta: float, device=None) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))


def mrope_axis_of_channel(head_dim: int, sections: Sequence[int], layout: str) -> torch.Tensor:
    """For each of the head_dim channels: which position axis (0=t, 1=h, 2=w) supplies its angle.

    ``hf``: split channels as sections*2 = [t,h,w,t,h,w] (so channel d and d+hd/2 share an axis).
    ``wallx_cuda``: contiguous [2t | 2h | 2w] (the reference's CUDA kernel; pairs can mix axes).
    """
    half = head_dim // 2
    assert sum(sections) == half
    if layout == "hf":
        ax = torch.cat([torch.full((s,), i, dtype=torch.long) for i, s in enumerate(sections)])
        return torch.cat([ax, ax])
    if layout == "wallx_cuda":
        return torch.cat([torch.full((2 * s,), i, dtype=torch.long) for i, s in enumerate(sections)])
    raise ValueError(layout)


def mrope_cos_sin(pos3: torch.Tensor, inv_freq: torch.Tensor, sections: Sequence[int], layout: str = "hf",
                  scaling: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """pos3 ``[3, T]`` -> per-token ``cos, sin`` of shape ``[T, head_dim]`` (fp32), axis-selected."""
    half = inv_freq.numel()
    hd = 2 * half
    freqs = pos3.float().unsqueeze(-1) * inv_freq.float().view(1, 1, half)  # [3, T, half]
    emb = torch.cat([freqs, freqs], dim=-1)  # [3, T, hd]
    ax = mrope_axis_of_channel(hd, sections, layout).to(pos3.device)
    sel = emb.gather(0, ax.view(1, 1, hd).expand(1, emb.shape[1], hd)).squeeze(0)  # [T, hd]
    return sel.cos() * scaling, sel.sin() * scaling


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x ``[T, heads, hd]``; cos/sin ``[T, hd]``; rotate-half form; computed in fp32."""
    xf = x.float()
    out = xf * cos.unsqueeze(1) + rotate_half(xf) * sin.unsqueeze(1)
    return out.to(x.dtype)


# ----------------------------------------------------------------------------- index generation
def rope_index(input_ids: torch.Tensor, image_grid_thw: Optional[torch.Tensor], video_grid_thw: Optional[torch.Tensor],
               second_per_grid_ts: Optional[torch.Tensor], attention_mask: Optional[torch.Tensor], spatial_merge_size: int,
               image_token_id: int, video_token_id: int, vision_start_token_id: int,
               tokens_per_second: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Position ids ``[3, B, S]`` (t/h/w) and ``mrope_deltas [B, 1]``; HF semantics (padding -> 1)."""
    B, S = input_ids.shape
    dev = input_ids.device
    if image_grid_thw is None and video_grid_thw is None:
        if attention_mask is not None:
            pos = attention_mask.long().cumsum(-1) - 1
            pos = pos.masked_fill(attention_mask == 0, 1)
            pos3 = pos.unsqueeze(0).expand(3, -1, -1).contiguous()
            mx = pos3.max(0)[0].max(-1, keepdim=True)[0]
            return pos3, mx + 1 - S
        pos3 = torch.arange(S, device=dev).view(1, 1, -1).expand(3, B, -1).contiguous()
        return pos3, torch.zeros((B, 1), dtype=input_ids.dtype, device=dev)
    if attention_mask is None:
        attention_mask = torch.ones_like(input_ids)
    ids_cpu = input_ids.cpu()
    am_cpu = attention_mask.cpu()
    img = image_grid_thw.cpu().tolist() if image_grid_thw is not None else []
    vid = video_grid_thw.cpu().tolist() if video_grid_thw is not None else []
    spg = second_per_grid_ts.cpu().tolist() if second_per_grid_ts is not None else None
    pos = torch.ones((3, B, S), dtype=torch.long)
    deltas = []
    ii = vi = 0
    for b in range(B):
        keep = am_cpu[b] == 1
        toks = ids_cpu[b][keep].tolist()
        n = len(toks)
        out = [[], [], []]
        st = 0
        nxt = 0
        # vision items are recognised as in the reference: the token after <vision_start>
        n_img = sum(1 for i in range(n - 1) if toks[i] == vision_start_token_id and toks[i + 1] == image_token_id)
        n_vid = sum(1 for i in range(n - 1) if toks[i] == vision_start_token_id and toks[i + 1] == video_token_id)
        rem_i, rem_v = n_img, n_vid
        for _ in range(n_img + n_vid):
            ed_i = toks.index(image_token_id, st) if (rem_i > 0 and image_token_id in toks[st:]) else n + 1
            ed_v = toks.index(video_token_id, st) if (rem_v > 0 and video_token_id in toks[st:]) else n + 1
            if ed_i < ed_v:
                t, h, w = img[ii]
                sec = 0.0
                ii += 1
                rem_i -= 1
                ed = ed_i
            else:
                t, h, w = vid[vi]
                sec = float(spg[vi]) if spg is not None else 1.0
                vi += 1
                rem_v -= 1
                ed = ed_v
            gh, gw = h // spatial_merge_size, w // spatial_merge_size
            text_len = ed - st
            for a in range(3):
                out[a].extend(range(nxt, nxt + text_len))
            base = nxt + text_len
            tmax = 0
            for ti in range(t):
                tv = int(ti * sec * tokens_per_second)
                tmax = max(tmax, tv)
                for hi in range(gh):
                    for wi in range(gw):
                        out[0].append(base + tv)
                        out[1].append(base + hi)
                        out[2].append(base + wi)
            nxt = base + max(tmax, gh - 1, gw - 1) + 1
            st = ed + t * gh * gw
        if st < n:
            for a in range(3):
                out[a].extend(range(nxt, nxt + n - st))
            nxt = nxt + n - st
        p = torch.tensor(out, dtype=torch.long)
        pos[:, b, keep] = p
        deltas.append(int(p.max().item()) + 1 - S if n > 0 else 0)
    return pos.to(dev), torch.tensor(deltas, dtype=torch.long, device=dev).unsqueeze(1)


def rot_pos_ids(grid_thw: Sequence[Sequence[int]], merge: int) -> torch.Tensor:
    """(h, w) patch coordinates ``[N, 2]`` in merge-block token order for every image."""
    out = []
    for t, h, w in grid_thw:
        hp = torch.arange(h).unsqueeze(1).expand(-1, w)
        wp = torch.arange(w).unsqueeze(0).expand(h, -1)
        hp = hp.reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).flatten()
        wp = wp.reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).flatten()
        out.append(torch.stack([hp, wp], dim=-1).repeat(t, 1))
    return torch.cat(out, dim=0)


def rot_pos_emb(inv_freq: torch.Tensor, grid_thw: Sequence[Sequence[int]], merge: int) -> torch.Tensor:
    """ViT rotary angle table ``[N, 2 * len(inv_freq)]`` = ``[h_pos * f | w_pos * f]``."""
    ids = rot_pos_ids(grid_thw, merge).to(inv_freq.device)
    ang = ids.float().unsqueeze(-1) * inv_freq.float().view(1, 1, -1)
    return ang.flatten(1)


def window_index(grid_thw: Sequence[Sequence[int]], window_size: int, merge: int, patch: int) -> Tuple[torch.Tensor, List[int]]:
    """Window permutation over merged tokens and ``cu_window_seqlens`` (in patches, x merge^2)."""
    unit = merge * merge
    vw = window_size // merge // patch
    index_all, cu = [], [0]
    base = 0
    for t, h, w in grid_thw:
        gh, gw = h // merge, w // merge
        idx = torch.arange(t * gh * gw).reshape(t, gh, gw)
        pad_h = vw - gh % vw
        pad_w = vw - gw % vw
        nh, nw = (gh + pad_h) // vw, (gw + pad_w) // vw
        pad = F.pad(idx, (0, pad_w, 0, pad_h), "constant", -100)
        pad = pad.reshape(t, nh, vw, nw, vw).permute(0, 1, 3, 2, 4).reshape(t, nh * nw, vw, vw)
        seqlens = (pad != -100).sum([2, 3]).reshape(-1)
        flat = pad.reshape(-1)
        index_all.append(flat[flat != -100] + base)
        cs = seqlens.cumsum(0) * unit + cu[-1]
        cu.extend(cs.tolist())
        base += t * gh * gw
    return torch.cat(index_all, dim=0), cu


def full_cu_seqlens(grid_thw: Sequence[Sequence[int]]) -> List[int]:
    cu = [0]
    for t, h, w in grid_thw:
        for _ in range(t):
            cu.append(cu[-1] + h * w)
    return cu


# ----------------------------------------------------------------------------- token routing
def route_plan(token_types: torch.Tensor, num_experts: int, align: int = 128):
    """Stable grouping of tokens by expert id.

    Returns ``(dest, seg)``: ``dest[t]`` is the row of token ``t`` in the grouped buffer, where
    expert ``e`` occupies rows ``[seg[e, 0], seg[e, 0] + seg[e, 1])`` and every segment start is a
    multiple of ``align`` (the padding rows are zero). ``seg[e, 2]`` is the padded row count.
    """
    tt = token_types.reshape(-1).long()
    T = tt.numel()
    dest = torch.empty(T, dtype=torch.long, device=tt.device)
    seg = torch.zeros((num_experts, 3), dtype=torch.long, device=tt.device)
    start = 0
    for e in range(num_experts):
        m = tt == e
        cnt = int(m.sum().item())
        dest[m] = start + torch.arange(cnt, device=tt.device)
        padded = (cnt + align - 1) // align * align
        seg[e, 0], seg[e, 1], seg[e, 2] = start, cnt, padded
        start += padded
    return dest, seg


def permute_rows(x: torch.Tensor, dest: torch.Tensor, total_rows: int) -> torch.Tensor:
    out = x.new_zeros((total_rows, x.shape[-1]))
    out.index_copy_(0, dest, x)
    return out


def unpermute_rows(y: torch.Tensor, dest: torch.Tensor) -> torch.Tensor:
    return y.index_select(0, dest)


# ----------------------------------------------------------------------------- attention
def attention_mask_varlen(cu_seqlens: Sequence[int], causal: bool, bidir: Optional[torch.Tensor], device) -> torch.Tensor:
    """Boolean ``[T, T]`` mask (True = may attend) for packed sequences."""
    T = cu_seqlens[-1]
    seq_id = torch.zeros(T, dtype=torch.long, device=device)
    for i in range(len(cu_seqlens) - 1):
        seq_id[cu_seqlens[i]:cu_seqlens[i + 1]] = i
    same = seq_id.unsqueeze(0) == seq_id.unsqueeze(1)
    if not causal:
        return same
    ar = torch.arange(T, device=device)
    allow = ar.unsqueeze(0) <= ar.unsqueeze(1)  # key index <= query index
    if bidir is not None:
        b = bidir.reshape(-1).bool()
        allow = allow | (b.unsqueeze(0) & b.unsqueeze(1))
    return same & allow


def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: Sequence[int], causal: bool,
                     bidir: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
    """q ``[T, Hq, D]``, k/v ``[T, Hkv, D]`` packed; returns ``[T, Hq, D]``. fp32 softmax."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    mask = attention_mask_varlen(list(cu_seqlens), causal, bidir, q.device)
    kk = k.repeat_interleave(rep, dim=1) if rep > 1 else k
    vv = v.repeat_interleave(rep, dim=1) if rep > 1 else v
    s = torch.einsum("qhd,khd->hqk", q.float(), kk.float()) * scale
    s = s.masked_fill(~mask.unsqueeze(0), float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vv.float()).to(q.dtype)


def attention_prefix(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, k_new: torch.Tensor,
                     v_new: torch.Tensor, causal_new: bool, scale: Optional[float] = None) -> torch.Tensor:
    """Queries ``[B, Sq, Hq, D]`` attend to a cached prefix ``[B, Sp, Hkv, D]`` plus their own keys.

    ``causal_new=False``: the new tokens see each other in both directions (action block).
    """
    B, Sq, Hq, D = q.shape
    Hkv = k_new.shape[2]
    rep = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    kk = torch.cat([k_cache, k_new], dim=1)
    vv = torch.cat([v_cache, v_new], dim=1)
    if rep > 1:
        kk = kk.repeat_interleave(rep, dim=2)
        vv = vv.repeat_interleave(rep, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kk.float()) * scale
    if causal_new:
        Sp = k_cache.shape[1]
        ar_q = torch.arange(Sq, device=q.device).unsqueeze(1) + Sp
        ar_k = torch.arange(Sp + Sq, device=q.device).unsqueeze(0)
        s = s.masked_fill(~(ar_k <= ar_q).view(1, 1, Sq, Sp + Sq), float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhqk,bkhd->bqhd", p, vv.float()).to(q.dtype)


# ----------------------------------------------------------------------------- losses / optimiser
def lm_head_ce(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100):
    """Per-row CE (0 at ignored rows) and argmax prediction; hidden ``[R, H]``, labels ``[R]``."""
    logits = F.linear(hidden, weight)
    loss = F.cross_entropy(logits.float(), labels, ignore_index=ignore_index, reduction="none")
    return loss, logits.argmax(-1)


def adamw_step(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, step: int, lr: float, beta1: float,
               beta2: float, eps: float, weight_decay: float, grad_scale: float = 1.0) -> None:
    """Decoupled-weight-decay Adam on fp32 master ``p`` in place (torch.optim.AdamW semantics)."""
    g = g.float() * grad_scale
    p.mul_(1.0 - lr * weight_decay)
    m.mul_(beta1).add_(g, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)

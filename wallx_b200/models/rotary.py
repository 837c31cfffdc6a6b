"""Rotary-embedding modules and helpers under the names of the reference's model file.

The model itself never calls these: positions are turned into per-token cos / sin tables once per
step and the rotation runs inside ``rope_qk`` on the packed QKV buffer. They exist for code that
imports the building blocks (wall_x/model/qwen2_5_based/modeling_qwen2_5_vl.py:
``Qwen2_5_VisionRotaryEmbedding`` :108-119, ``Qwen2_5_VLRotaryEmbedding`` :635-712,
``rotate_half`` :723, ``apply_multimodal_rotary_pos_emb`` :731-773, ``apply_rotary_pos_emb_vision``
:222-233, ``apply_rotary_pos_emb_flashatt`` :158-165, ``repeat_kv`` :776) and as plain-PyTorch
oracles in tests.
"""
from __future__ import annotations

from typing import Sequence, Tuple

import torch
import torch.nn as nn

from ..ops import ref


class Qwen2_5_VisionRotaryEmbedding(nn.Module):
    """Angle table of the vision tower: ``forward(n)`` -> ``[n, dim / 2]`` = position x inverse frequency."""

    def __init__(self, dim: int, theta: float = 10000.0):
        super().__init__()
        self.register_buffer("inv_freq", 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim)), persistent=False)

    def forward(self, seqlen: int) -> torch.Tensor:
        pos = torch.arange(seqlen, device=self.inv_freq.device, dtype=self.inv_freq.dtype)
        return torch.outer(pos, self.inv_freq)


class Qwen2_5_VLRotaryEmbedding(nn.Module):
    """3-axis tables of the language model: ``forward(x, position_ids [3, B, S])`` -> ``cos, sin [3, B, S, head_dim]``
    in ``x.dtype``, computed in fp32; ``attention_scaling`` is 1 for the default rope type."""

    def __init__(self, config=None, device=None, head_dim: int = 0, rope_theta: float = 0.0):
        super().__init__()
        if config is not None:
            head_dim = int(getattr(config, "head_dim", 0) or config.hidden_size // config.num_attention_heads)
            rope_theta = float(getattr(config, "rope_theta", 1e6))
        self.attention_scaling = 1.0
        self.register_buffer("inv_freq", ref.rope_inv_freq(head_dim, rope_theta, device=device), persistent=False)

    @torch.no_grad()
    def forward(self, x: torch.Tensor, position_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        freqs = position_ids.to(self.inv_freq.device).float().unsqueeze(-1) * self.inv_freq.view(1, 1, 1, -1)
        emb = torch.cat((freqs, freqs), dim=-1)
        return (emb.cos() * self.attention_scaling).to(x.dtype), (emb.sin() * self.attention_scaling).to(x.dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    return ref.rotate_half(x)


def apply_multimodal_rotary_pos_emb(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                                    mrope_section: Sequence[int], unsqueeze_dim: int = 1):
    """Hugging Face layout: the channel halves are split as ``mrope_section * 2`` and chunk i takes axis ``i % 3``.
    q / k ``[B, H, S, D]``, cos / sin ``[3, B, S, D]``."""
    D = q.shape[-1]
    ax = ref.mrope_axis_of_channel(D, list(mrope_section), "hf").to(cos.device)
    sel = ax.view(1, 1, 1, D).expand(1, *cos.shape[1:])
    c = cos.gather(0, sel).squeeze(0).unsqueeze(unsqueeze_dim)
    s = sin.gather(0, sel).squeeze(0).unsqueeze(unsqueeze_dim)
    return q * c + ref.rotate_half(q) * s, k * c + ref.rotate_half(k) * s


def apply_rotary_pos_emb_vision(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """q / k ``[S, H, D]``, cos / sin ``[S, D]``; computed in fp32 and cast back."""
    c, s = cos.unsqueeze(-2).float(), sin.unsqueeze(-2).float()
    qf, kf = q.float(), k.float()
    return (qf * c + ref.rotate_half(qf) * s).to(q.dtype), (kf * c + ref.rotate_half(kf) * s).to(k.dtype)


def apply_rotary_pos_emb_flashatt(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """Same rotation for ``[..., S, H, D]`` inputs with full-width tables (the first half of cos / sin is what
    the reference hands to flash-attn's rotary kernel; both halves are equal)."""
    return apply_rotary_pos_emb_vision(q, k, cos, sin)


def repeat_kv(hidden_states: torch.Tensor, n_rep: int) -> torch.Tensor:
    """``[B, Hkv, S, D]`` -> ``[B, Hkv * n_rep, S, D]`` (each KV head repeated for its query group). The attention
    kernels index the shared KV head instead of materialising this."""
    if n_rep == 1:
        return hidden_states
    B, H, S, D = hidden_states.shape
    return hidden_states[:, :, None].expand(B, H, n_rep, S, D).reshape(B, H * n_rep, S, D)

"""Qwen2.5-VL vision tower on the packed-token operator layer.

Behaviour follows the reference's ``Qwen2_5_VisionTransformerPretrainedModel``
(modeling_qwen2_5_vl.py:440-632): Conv3d patch embedding (kernel = stride, i.e. a GEMM), 2-D
rotary angles in merge-block order, window re-ordering, window attention in all blocks except
``fullatt_block_indexes``, RMSNorm + biased SwiGLU MLP, patch merger (RMSNorm -> Linear -> GELU ->
Linear) and the inverse re-ordering. Index tables (rotary ids, window permutation, cu_seqlens)
are functions of ``grid_thw`` only, which lives on the host, so they are computed without any
device synchronisation and cached per grid signature.
"""
from __future__ import annotations

from typing import Dict, Sequence, Tuple

import torch
import torch.nn as nn

from ..config import Qwen2_5_VLVisionConfig
from ..ops import blocks as BK
from ..ops import functional as F_
from ..ops import ref
from ..ops import index as IX
from .layers import Linear, RMSNorm, SwiGLUFFN


class VisionPatchEmbed(nn.Module):
    def __init__(self, patch_size: int, temporal_patch_size: int, in_channels: int, embed_dim: int):
        super().__init__()
        self.in_dim = in_channels * temporal_patch_size * patch_size * patch_size
        self.embed_dim = embed_dim
        self.shape5 = (embed_dim, in_channels, temporal_patch_size, patch_size, patch_size)
        # parameter keeps the Conv3d weight shape of the checkpoint: visual.patch_embed.proj.weight
        self.proj = nn.Module()
        self.proj.weight = nn.Parameter(torch.empty(self.shape5))

    def forward(self, patches: torch.Tensor) -> torch.Tensor:
        w = self.proj.weight.view(self.embed_dim, self.in_dim)
        return F_.linear(patches.to(w.dtype), w, None)


class VisionAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = dim // num_heads
        self.qkv = Linear(dim, dim * 3, bias=True)
        self.proj = Linear(dim, dim, bias=True)

    def forward(self, x, meta: F_.AttnMeta, cos, sin, residual):
        qkv = self.qkv(x)
        qkv = F_.rope_qk(qkv, cos, sin, 2 * self.num_heads, self.head_dim)
        o = F_.attention_packed(qkv, meta, self.num_heads, self.num_heads, self.head_dim)
        return self.proj(o, residual=residual)


class VisionBlock(nn.Module):
    def __init__(self, config: Qwen2_5_VLVisionConfig):
        super().__init__()
        self.norm1 = RMSNorm(config.hidden_size, eps=1e-6)
        self.norm2 = RMSNorm(config.hidden_size, eps=1e-6)
        self.attn = VisionAttention(config.hidden_size, config.num_heads)
        self.mlp = SwiGLUFFN(config.hidden_size, config.intermediate_size, bias=True)

    def forward(self, x, meta, cos, sin):
        a, f = self.attn, self.mlp
        if BK.usable(x) and type(a.qkv) is Linear and type(a.proj) is Linear and type(f) is SwiGLUFFN:
            # the whole block, forward or backward, is one host call (csrc/blocks.cpp)
            return BK.transformer_block(x, self.norm1.weight, a.qkv.weight, a.qkv.bias, a.proj.weight, a.proj.bias,
                                        self.norm2.weight, list(f.weights()), f.gate_up_bias, f.down_bias, meta=meta,
                                        cos=cos, sin=sin, n_rot=2 * a.num_heads, hq=a.num_heads, hkv=a.num_heads,
                                        d=a.head_dim, eps=self.norm1.variance_epsilon)
        x = self.attn(self.norm1(x), meta, cos, sin, residual=x)
        return self.mlp(self.norm2(x), residual=x)


class PatchMerger(nn.Module):
    def __init__(self, dim: int, context_dim: int, spatial_merge_size: int = 2):
        super().__init__()
        self.hidden_size = context_dim * (spatial_merge_size ** 2)
        self.ln_q = RMSNorm(context_dim, eps=1e-6)
        self.mlp = nn.ModuleList([Linear(self.hidden_size, self.hidden_size), nn.Identity(), Linear(self.hidden_size, dim)])

    def forward(self, x):
        x = self.ln_q(x).view(-1, self.hidden_size)
        x = F_.linear_gelu(x, self.mlp[0].weight, self.mlp[0].bias)
        return self.mlp[2](x)


class VisionTables:
    """Host-computed, device-resident index tables for one ``grid_thw`` signature."""

    def __init__(self, grid: Sequence[Sequence[int]], cfg: Qwen2_5_VLVisionConfig, inv_freq: torch.Tensor, device):
        merge, unit = cfg.spatial_merge_size, cfg.spatial_merge_size ** 2
        win_idx, cu_win = IX.window_index(grid, cfg.window_size, merge, cfg.patch_size)
        # drop empty windows (duplicate offsets)
        cu_win_u = [cu_win[0]] + [c for p, c in zip(cu_win[:-1], cu_win[1:]) if c != p]
        cu_full = ref.full_cu_seqlens(grid)
        angles = IX.rot_pos_emb(inv_freq.cpu(), grid, merge)  # [N, hd/2]
        n = angles.shape[0]
        patch_perm = (win_idx.view(-1, 1) * unit + torch.arange(unit).view(1, -1)).reshape(-1)  # [N]
        angles = angles[patch_perm]
        emb = torch.cat([angles, angles], dim=-1)
        self.n_patches = n
        self.patch_perm = patch_perm.to(device)
        self.reverse = torch.argsort(win_idx).to(device)
        self.cos = emb.cos().contiguous().to(device)
        self.sin = emb.sin().contiguous().to(device)
        self.meta_window = F_.AttnMeta(cu_win_u, device, causal=False)
        self.meta_full = F_.AttnMeta(cu_full, device, causal=False)


class VisionTransformer(nn.Module):
    def __init__(self, config: Qwen2_5_VLVisionConfig):
        super().__init__()
        self.config = config
        self.spatial_merge_size = config.spatial_merge_size
        self.patch_size = config.patch_size
        self.fullatt_block_indexes = list(config.fullatt_block_indexes)
        self.window_size = config.window_size
        self.spatial_merge_unit = config.spatial_merge_size ** 2
        self.patch_embed = VisionPatchEmbed(config.patch_size, config.temporal_patch_size, config.in_channels,
                                            config.hidden_size)
        head_dim = config.hidden_size // config.num_heads
        inv_freq = 1.0 / (10000.0 ** (torch.arange(0, head_dim // 2, 2, dtype=torch.float) / (head_dim // 2)))
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self.blocks = nn.ModuleList([VisionBlock(config) for _ in range(config.depth)])
        self.merger = PatchMerger(config.out_hidden_size, config.hidden_size, config.spatial_merge_size)
        self._tables: Dict[Tuple, VisionTables] = {}

    @property
    def dtype(self):
        return self.patch_embed.proj.weight.dtype

    def tables(self, grid_thw, device) -> VisionTables:
        grid = grid_thw.tolist() if isinstance(grid_thw, torch.Tensor) else [list(g) for g in grid_thw]
        key = (tuple(tuple(int(v) for v in g) for g in grid), str(device))
        t = self._tables.get(key)
        if t is None:
            if len(self._tables) > 64:
                self._tables.clear()
            t = VisionTables([list(k) for k in key[0]], self.config, self.inv_freq.float(), device)
            self._tables[key] = t
        return t

    def forward(self, patches: torch.Tensor, grid_thw, grid_host=None) -> torch.Tensor:
        """patches ``[N, C*2*14*14]``; returns merged tokens ``[N / merge^2, out_hidden]``.

        ``grid_host`` (a list of ``(t, h, w)``) avoids reading ``grid_thw`` back from the device.
        """
        tb = self.tables(grid_host if grid_host is not None else grid_thw, patches.device)
        x = self.patch_embed(patches)
        x = x.index_select(0, tb.patch_perm)
        for i, blk in enumerate(self.blocks):
            meta = tb.meta_full if i in self.fullatt_block_indexes else tb.meta_window
            x = blk(x, meta, tb.cos, tb.sin)
        x = self.merger(x)
        return x.index_select(0, tb.reverse)

"""Low-rank adapters on named projections (the subset of peft the reference uses,
modeling_qwen2_5_vl_act.py:880-903: ``LoraConfig(r, lora_alpha, target_modules, lora_dropout,
bias="none")`` applied to the language model).

Target names follow the reference's module names (``q_proj``, ``k_proj``, ``v_proj``, ``o_proj``,
``gate_proj``, ``up_proj``, ``down_proj``). Because q/k/v and gate/up are fused here, an adapter on
``q_proj`` is an adapter on the q rows of the fused projection: ``y += scale * B(A(drop(x)))`` is
added to the matching output columns. Base weights are frozen, as peft does.
"""
from __future__ import annotations

import math
from typing import List, Tuple

import torch
import torch.nn as nn

from .layers import FusedQKV, Linear


class LoRAAdapter(nn.Module):
    def __init__(self, in_features: int, out_features: int, r: int, alpha: float, dropout: float):
        super().__init__()
        self.lora_A = nn.Parameter(torch.empty(r, in_features))
        self.lora_B = nn.Parameter(torch.zeros(out_features, r))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.scaling = alpha / r
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    def forward(self, x):
        # rank is small (not a multiple of 8 in general): plain matmuls, negligible cost
        h = torch.nn.functional.linear(self.dropout(x), self.lora_A.to(x.dtype))
        return torch.nn.functional.linear(h, self.lora_B.to(x.dtype)) * self.scaling


class LoRALinear(nn.Module):
    """Wraps a :class:`Linear`; the wrapped weight is frozen."""

    def __init__(self, base: Linear, r: int, alpha: float, dropout: float):
        super().__init__()
        self.base = base
        for p in base.parameters():
            p.requires_grad_(False)
        self.adapter = LoRAAdapter(base.in_features, base.out_features, r, alpha, dropout)
        self.adapter.to(base.weight.device)

    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return self.base.bias

    def forward(self, x, residual=None):
        return self.base(x, residual=residual) + self.adapter(x)


class LoRAFusedQKV(nn.Module):
    def __init__(self, base: FusedQKV, which: List[str], r: int, alpha: float, dropout: float):
        super().__init__()
        self.base = base
        for p in base.parameters():
            p.requires_grad_(False)
        sizes = {"q_proj": base.q_out, "k_proj": base.kv_out, "v_proj": base.kv_out}
        self.offsets = {"q_proj": 0, "k_proj": base.q_out, "v_proj": base.q_out + base.kv_out}
        self.adapters = nn.ModuleDict({n: LoRAAdapter(base.hidden, sizes[n], r, alpha, dropout) for n in which})
        self.adapters.to(base.weight.device)
        self.sizes = sizes

    def forward(self, x):
        y = self.base(x)
        parts = []
        for n in ("q_proj", "k_proj", "v_proj"):
            if n in self.adapters:
                parts.append(self.adapters[n](x))
            else:
                parts.append(y.new_zeros(y.shape[:-1] + (self.sizes[n],)))
        return y + torch.cat(parts, dim=-1)


def apply_lora(model: nn.Module, r: int = 8, alpha: float = 32, target_modules=("q_proj", "v_proj"),
               dropout: float = 0.1) -> int:
    """Freeze ``model`` and add adapters to the requested projections. Returns how many modules were wrapped."""
    for p in model.parameters():
        p.requires_grad_(False)
    n = 0
    targets = set(target_modules)
    for name, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            if isinstance(child, FusedQKV):
                which = [t for t in ("q_proj", "k_proj", "v_proj") if t in targets]
                if which:
                    setattr(mod, child_name, LoRAFusedQKV(child, which, r, alpha, dropout))
                    n += len(which)
            elif isinstance(child, Linear) and child_name in targets:
                setattr(mod, child_name, LoRALinear(child, r, alpha, dropout))
                n += 1
    return n


def print_trainable_parameters(model: nn.Module) -> Tuple[int, int]:
    tr = sum(p.numel() for p in model.parameters() if p.requires_grad)
    al = sum(p.numel() for p in model.parameters())
    print(f"trainable params: {tr:,} || all params: {al:,} || trainable%: {100 * tr / max(al, 1):.4f}")
    return tr, al

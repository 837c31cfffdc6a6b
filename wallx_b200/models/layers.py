"""Building blocks with B200-first parameter layouts and HF-compatible state dicts.

Internally q/k/v are one weight, gate/up are one weight interleaved in 16-row blocks (so SwiGLU
runs in the GEMM epilogue), and FFN widths are padded to a multiple of 16. ``state_dict()`` and
``load_state_dict()`` still speak the reference's key layout (``q_proj/k_proj/v_proj``,
``gate_proj/up_proj/down_proj``; modeling_qwen2_5_vl.py:54-67, 821-832 and
modeling_qwen2_5_vl_act.py:67-82) through state-dict hooks.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as F_
from ..ops import ref


def round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.variance_epsilon = eps

    def forward(self, x, dest=None, out_rows: int = 0):
        return F_.rms_norm(x, self.weight, self.variance_epsilon, dest, out_rows)

    def extra_repr(self):
        return f"{tuple(self.weight.shape)}, eps={self.variance_epsilon}"


class Linear(nn.Module):
    """nn.Linear-compatible parameters (``weight [out, in]``, optional ``bias``) on our GEMM."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None

    def forward(self, x, residual=None):
        return F_.linear(x, self.weight, self.bias, residual)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


class FusedQKV(nn.Module):
    """One ``[(Hq + 2 Hkv) * D, hidden]`` projection; state dict exposes q_proj/k_proj/v_proj."""

    def __init__(self, hidden: int, q_out: int, kv_out: int, bias: bool = True):
        super().__init__()
        self.hidden, self.q_out, self.kv_out = hidden, q_out, kv_out
        self.weight = nn.Parameter(torch.empty(q_out + 2 * kv_out, hidden))
        self.bias = nn.Parameter(torch.zeros(q_out + 2 * kv_out)) if bias else None
        self._register_state_dict_hook(FusedQKV._split_hook)

    def forward(self, x):
        return F_.linear(x, self.weight, self.bias)

    # parent modules name this submodule "qkv_proj"; keys are rewritten relative to the parent
    @staticmethod
    def _split_hook(module, state_dict, prefix, local_metadata):
        parent = prefix[: -len("qkv_proj.")] if prefix.endswith("qkv_proj.") else None
        if parent is None:
            return
        sizes = [module.q_out, module.kv_out, module.kv_out]
        for kind in ("weight", "bias"):
            key = prefix + kind
            if key not in state_dict:
                continue
            parts = state_dict.pop(key).split(sizes, dim=0)
            for name, part in zip(("q_proj", "k_proj", "v_proj"), parts):
                state_dict[f"{parent}{name}.{kind}"] = part.clone()

    @staticmethod
    def merge_hook_for_parent(name: str = "qkv_proj"):
        """Load-time hook to register on the *parent* module: torch hands a child only the keys
        under the child's own prefix, and q_proj/k_proj/v_proj live beside it, not under it."""

        def hook(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
            for kind in ("weight", "bias"):
                keys = [f"{prefix}{n}.{kind}" for n in ("q_proj", "k_proj", "v_proj")]
                if all(k in state_dict for k in keys):
                    state_dict[f"{prefix}{name}.{kind}"] = torch.cat([state_dict.pop(k) for k in keys], dim=0)

        return hook


class SwiGLUFFN(nn.Module):
    """``down(silu(gate(x)) * up(x))`` with a fused, interleaved, 16-padded gate/up weight.

    ``gate_up.weight`` is ``[2 Ip, hidden]`` in blocks ``[16 gate rows | 16 up rows]``; ``down`` is
    ``[hidden, Ip]``. Padding rows/columns are zero and stay zero under training (their gradients
    are exactly zero). The state dict shows ``gate_proj/up_proj/down_proj`` at the logical width.
    """

    def __init__(self, hidden: int, intermediate: int, bias: bool = False):
        super().__init__()
        self.hidden, self.intermediate = hidden, intermediate
        # widths are padded so that every row pitch is a multiple of 128 B (TMA, 128B swizzle)
        self.padded = round_up(intermediate, 64)
        self.gate_up_weight = nn.Parameter(torch.empty(2 * self.padded, hidden))
        self.down_weight = nn.Parameter(torch.empty(hidden, self.padded))
        if bias:
            self.gate_up_bias = nn.Parameter(torch.zeros(2 * self.padded))
            self.down_bias = nn.Parameter(torch.zeros(hidden))
        else:
            self.gate_up_bias = None
            self.down_bias = None
        self._register_state_dict_hook(SwiGLUFFN._split_hook)
        self._register_load_state_dict_pre_hook(self._merge_hook)

    def forward(self, x, residual=None):
        return F_.swiglu_ffn(x, self.gate_up_weight, self.gate_up_bias, self.down_weight, self.down_bias, residual)

    def weights(self):
        return self.gate_up_weight, self.down_weight

    # ---- layout conversion
    def pack_gate_up(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        pad = self.padded - self.intermediate
        if pad:
            z = gate.new_zeros((pad,) + tuple(gate.shape[1:]))
            gate, up = torch.cat([gate, z]), torch.cat([up, z])
        return ref.interleave_gate_up(gate, up, 16)

    def unpack_gate_up(self, gu: torch.Tensor):
        g, u = ref.deinterleave_gate_up(gu, 16, dim=0)
        return g[: self.intermediate].clone(), u[: self.intermediate].clone()

    @staticmethod
    def _split_hook(module, state_dict, prefix, local_metadata):
        k = prefix + "gate_up_weight"
        if k in state_dict:
            g, u = module.unpack_gate_up(state_dict.pop(k))
            state_dict[prefix + "gate_proj.weight"] = g
            state_dict[prefix + "up_proj.weight"] = u
        k = prefix + "down_weight"
        if k in state_dict:
            state_dict[prefix + "down_proj.weight"] = state_dict.pop(k)[:, : module.intermediate].clone()
        k = prefix + "gate_up_bias"
        if k in state_dict:
            g, u = module.unpack_gate_up(state_dict.pop(k))
            state_dict[prefix + "gate_proj.bias"] = g
            state_dict[prefix + "up_proj.bias"] = u
        k = prefix + "down_bias"
        if k in state_dict:
            state_dict[prefix + "down_proj.bias"] = state_dict.pop(k)

    def _merge_hook(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        gk, uk, dk = prefix + "gate_proj.weight", prefix + "up_proj.weight", prefix + "down_proj.weight"
        if gk in state_dict and uk in state_dict:
            state_dict[prefix + "gate_up_weight"] = self.pack_gate_up(state_dict.pop(gk), state_dict.pop(uk))
        if dk in state_dict:
            d = state_dict.pop(dk)
            pad = self.padded - self.intermediate
            if pad:
                d = torch.cat([d, d.new_zeros((d.shape[0], pad))], dim=1)
            state_dict[prefix + "down_weight"] = d
        gk, uk, dk = prefix + "gate_proj.bias", prefix + "up_proj.bias", prefix + "down_proj.bias"
        if gk in state_dict and uk in state_dict:
            state_dict[prefix + "gate_up_bias"] = self.pack_gate_up(state_dict.pop(gk), state_dict.pop(uk))
        if dk in state_dict:
            state_dict[prefix + "down_bias"] = state_dict.pop(dk)

    @torch.no_grad()
    def reset_parameters(self, std: float, generator: Optional[torch.Generator] = None):
        g = torch.empty(self.intermediate, self.hidden).normal_(0.0, std, generator=generator)
        u = torch.empty(self.intermediate, self.hidden).normal_(0.0, std, generator=generator)
        d = torch.empty(self.hidden, self.intermediate).normal_(0.0, std, generator=generator)
        self.gate_up_weight.copy_(self.pack_gate_up(g, u))
        self.down_weight.zero_()
        self.down_weight[:, : self.intermediate].copy_(d)
        if self.gate_up_bias is not None:
            self.gate_up_bias.zero_()
            self.down_bias.zero_()

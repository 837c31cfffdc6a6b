"""Qwen2.5-VL language model with the dual-expert (token-type routed) FFN, on packed tokens.

Parity targets: ``Qwen2_5_VLAttention`` / ``Qwen2_5_VLFlashAttention2``
(modeling_qwen2_5_vl.py:790-1023), ``BlockSparseMLP`` / ``SparseMoeBlock`` /
``Qwen2_5_VLDecoderLayer_with_MoE`` / ``Qwen2_5_VLMoEModel`` (modeling_qwen2_5_vl_act.py:67-732) and
the plain ``Qwen2_5_VLDecoderLayer`` when ``mlp_moe`` is off.

Differences by design: activations are ``[T, hidden]`` with no padding rows; q/k/v come from one
GEMM; mRoPE cos/sin are computed once per step for all layers; the token-type permutation is a
routing plan computed once per batch and fused into the post-attention RMSNorm (gather) and the
down-projection epilogue (scatter + residual).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..config import Qwen2_5_VLConfig
from ..ops import blocks as BK
from ..ops import functional as F_
from ..ops import ref
from .generation import MoEModelMaskMixin
from .layers import FusedQKV, Linear, RMSNorm, SwiGLUFFN


class StepContext:
    """Everything the decoder layers share for one forward pass over packed tokens."""

    def __init__(self, meta: F_.AttnMeta, cos: torch.Tensor, sin: torch.Tensor, plan: Optional[F_.RoutePlan],
                 cache: Optional["KVCache"] = None, cache_mode: str = "none"):
        self.meta = meta
        self.cos, self.sin = cos, sin
        self.plan = plan
        self.cache = cache
        self.cache_mode = cache_mode  # "none" | "prefill" | "append"


class KVCache:
    """Per-layer packed K/V storage for the prefix-reusing denoise loop and token decoding.

    Layout: for each sample ``b`` a slot of ``capacity[b]`` rows in one ``[rows, 2 * Hkv * D]``
    buffer per layer (k columns then v columns). ``length[b]`` rows of each slot are valid.
    """

    def __init__(self, num_layers: int, capacities: Sequence[int], kv_width: int, device, dtype):
        self.capacities = [int(c) for c in capacities]
        self.offsets = [0]
        for c in self.capacities:
            self.offsets.append(self.offsets[-1] + c)
        rows = self.offsets[-1]
        self.kv_width = kv_width
        self.buffers = [torch.zeros((rows, 2 * kv_width), device=device, dtype=dtype) for _ in range(num_layers)]
        self.lengths = [0] * len(self.capacities)
        self.device = device

    @property
    def batch(self) -> int:
        return len(self.capacities)

    def slot_rows(self, b: int, start: int, n: int) -> torch.Tensor:
        base = self.offsets[b] + start
        return torch.arange(base, base + n, device=self.device)


class Attention(nn.Module):
    def __init__(self, config: Qwen2_5_VLConfig, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.num_key_value_heads
        self.head_dim = config.head_dim
        self.qkv_proj = FusedQKV(self.hidden_size, self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, bias=True)
        self.o_proj = Linear(self.num_heads * self.head_dim, self.hidden_size, bias=False)
        self._register_load_state_dict_pre_hook(FusedQKV.merge_hook_for_parent("qkv_proj"))

    def forward(self, x: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> torch.Tensor:
        hq, hkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = self.qkv_proj(x)
        cached = not (ctx.cache is None or ctx.cache_mode == "none")
        if cached and F_.cached_step_kernels_usable(qkv, d):
            # rotary and cache write in one launch, then the small-query kernel when only a few rows are new
            buf = ctx.cache.buffers[self.layer_idx]
            F_.rope_cache_(qkv, ctx.cos, ctx.sin, ctx.meta.cache_rows, buf, hq, hkv, d)
            o = F_.attention_decode(qkv[:, : hq * d], buf[:, : hkv * d], buf[:, hkv * d:], ctx.meta, hq, hkv, d)
            return self.o_proj(o, residual=residual)
        qkv = F_.rope_qk(qkv, ctx.cos, ctx.sin, hq + hkv, d)
        if not cached:
            o = F_.attention_packed(qkv, ctx.meta, hq, hkv, d)
        else:
            buf = ctx.cache.buffers[self.layer_idx]
            # write this call's k|v rows into their cache slots, then attend over the slots
            buf.index_copy_(0, ctx.meta.cache_rows, qkv[:, hq * d:])
            q = qkv[:, : hq * d]
            k = buf[:, : hkv * d]
            v = buf[:, hkv * d:]
            o = F_.attention(q, k, v, ctx.meta, hq, hkv, d)
        return self.o_proj(o, residual=residual)


class SparseMoeBlock(nn.Module):
    """Static experts selected by token type (no router); experts can have different widths."""

    def __init__(self, config: Qwen2_5_VLConfig, num_experts: int):
        super().__init__()
        self.num_experts = num_experts
        self.experts = nn.ModuleList(
            [SwiGLUFFN(int(config.experts[i]["hidden_size"]), int(config.experts[i]["intermediate_size"]), bias=False)
             for i in range(num_experts)])

    def forward(self, xp: torch.Tensor, residual: torch.Tensor, plan: F_.RoutePlan) -> torch.Tensor:
        return F_.moe_ffn(xp, residual, plan, [e.weights() for e in self.experts])


class DecoderLayer(nn.Module):
    def __init__(self, config: Qwen2_5_VLConfig, layer_idx: int):
        super().__init__()
        self.self_attn = Attention(config, layer_idx)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        if config.mlp_moe:
            self.moe = SparseMoeBlock(config, config.num_experts)
            self.mlp = None
        else:
            self.moe = None
            self.mlp = SwiGLUFFN(config.hidden_size, config.intermediate_size, bias=False)

    def _plain_modules(self) -> bool:
        """True when every projection is this package's own module (LoRA wrappers and the like take the
        operator-by-operator path)."""
        a = self.self_attn
        ok = type(a.qkv_proj) is FusedQKV and type(a.o_proj) is Linear
        if self.moe is not None:
            return ok and all(type(e) is SwiGLUFFN for e in self.moe.experts)
        return ok and type(self.mlp) is SwiGLUFFN

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        if BK.usable(x) and (ctx.cache is None or ctx.cache_mode == "none") and self._plain_modules():
            # the whole layer, forward or backward, is one host call (csrc/blocks.cpp)
            a = self.self_attn
            if self.moe is not None:
                ffn_w = [w for e in self.moe.experts for w in e.weights()]
                plan = ctx.plan
            else:
                ffn_w, plan = list(self.mlp.weights()), None
            return BK.transformer_block(
                x, self.input_layernorm.weight, a.qkv_proj.weight, a.qkv_proj.bias, a.o_proj.weight, a.o_proj.bias,
                self.post_attention_layernorm.weight, ffn_w, None, None, meta=ctx.meta, cos=ctx.cos, sin=ctx.sin,
                n_rot=a.num_heads + a.num_kv_heads, hq=a.num_heads, hkv=a.num_kv_heads, d=a.head_dim,
                eps=self.input_layernorm.variance_epsilon, plan=plan)
        x = self.self_attn(self.input_layernorm(x), ctx, residual=x)
        if self.moe is not None and ctx.plan.single_expert is not None and not torch.is_grad_enabled():
            # every token of this call belongs to one expert (known on the host): a plain FFN, no grouping of rows
            return self.moe.experts[ctx.plan.single_expert](self.post_attention_layernorm(x), residual=x)
        if self.moe is not None:
            xp = self.post_attention_layernorm(x, dest=ctx.plan.dest, out_rows=ctx.plan.rows)
            return self.moe(xp, x, ctx.plan)
        return self.mlp(self.post_attention_layernorm(x), residual=x)


class Qwen2_5_VLMoEModel(MoEModelMaskMixin, nn.Module):
    """Embedding, N decoder layers, final norm. ``forward`` works on packed embeddings."""

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str, num_experts: Optional[int] = None, *args, **kwargs):
        """Decoder stack from a checkpoint directory: ``config.json`` (or ``config=``), optionally with another
        number of experts, and the ``model.*`` tensors of its safetensors files; stock Qwen2.5-VL FFN keys are mapped
        onto expert 0 (reference: modeling_qwen2_5_vl_act.py:283-311)."""
        import os

        from ..train.checkpoint import load_safetensors_dir, rename_qwen_to_moe

        config = kwargs.get("config")
        if config is None:
            config = Qwen2_5_VLConfig.from_pretrained(os.path.join(pretrained_model_name_or_path, "config.json"))
        if num_experts is not None:
            config.num_experts = int(num_experts)
        model = cls(config)
        state = load_safetensors_dir(pretrained_model_name_or_path)
        if config.mlp_moe:
            state = rename_qwen_to_moe(state)
        own = {k[len("model."):]: v for k, v in state.items() if k.startswith("model.")}
        missing, unexpected = model.load_state_dict(own, strict=False)
        model._load_report = {"missing": list(missing), "unexpected": list(unexpected)}
        return model

    def __init__(self, config: Qwen2_5_VLConfig):
        super().__init__()
        self.config = config
        self.padding_idx = config.pad_token_id
        self.vocab_size = config.vocab_size
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, self.padding_idx)
        self.layers = nn.ModuleList([DecoderLayer(config, i) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        inv_freq = ref.rope_inv_freq(config.head_dim, config.rope_theta)
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self.gradient_checkpointing = False

    def get_input_embeddings(self):
        return self.embed_tokens

    def set_input_embeddings(self, value):
        self.embed_tokens = value

    def rotary(self, pos3: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """pos3 ``[3, T]`` -> fp32 cos/sin ``[T, head_dim]`` shared by every layer."""
        cos, sin = ref.mrope_cos_sin(pos3, self.inv_freq.float(), self.config.mrope_section, self.config.mrope_layout)
        return cos.contiguous(), sin.contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        for layer in self.layers:
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                x = torch.utils.checkpoint.checkpoint(layer, x, ctx, use_reentrant=False)
            else:
                x = layer(x, ctx)
        return self.norm(x)

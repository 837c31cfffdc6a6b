"""Model configuration (reads and writes the HF ``config.json`` of a Wall-X checkpoint verbatim).

Field names and defaults follow the reference's ``Qwen2_5_VLVisionConfig`` / ``Qwen2_5_VLConfig``
(wall_x/model/qwen2_5_based/configuration_qwen2_5_vl.py:5-40, 168-243), including the
``rope_scaling`` back-compat rewrite (``type: mrope`` -> ``default``). Framework-only keys
(``mrope_layout``, ``action_attn``) default to the reference behaviour of its non-flash path.
"""
from __future__ import annotations

import copy
import json
import os
from typing import Any, Dict, List


class _Base:
    def to_dict(self) -> Dict[str, Any]:
        out = {}
        for k, v in self.__dict__.items():
            if k.startswith("_"):
                continue
            out[k] = v.to_dict() if isinstance(v, _Base) else copy.deepcopy(v)
        return out

    def __repr__(self) -> str:
        return f"{type(self).__name__}({json.dumps(self.to_dict(), indent=1, default=str)})"

    def get(self, key, default=None):
        return getattr(self, key, default)


class Qwen2_5_VLVisionConfig(_Base):
    model_type = "qwen2_5_vl"

    def __init__(self, depth=32, hidden_size=3584, hidden_act="silu", intermediate_size=3420, num_heads=16,
                 in_channels=3, patch_size=14, spatial_merge_size=2, temporal_patch_size=2, tokens_per_second=4,
                 window_size=112, out_hidden_size=3584, fullatt_block_indexes=(7, 15, 23, 31), **kwargs):
        self.depth = depth
        self.hidden_size = hidden_size
        self.hidden_act = hidden_act
        self.intermediate_size = intermediate_size
        self.num_heads = num_heads
        self.in_channels = in_channels
        self.patch_size = patch_size
        self.spatial_merge_size = spatial_merge_size
        self.temporal_patch_size = temporal_patch_size
        self.tokens_per_second = tokens_per_second
        self.window_size = window_size
        self.out_hidden_size = out_hidden_size
        self.fullatt_block_indexes = list(fullatt_block_indexes)
        for k, v in kwargs.items():
            setattr(self, k, v)


class Qwen2_5_VLConfig(_Base):
    model_type = "qwen2_5_vl"
    # Kept as metadata only (the reference never activates them either).
    base_model_tp_plan = {
        "layers.*.self_attn.q_proj": "colwise",
        "layers.*.self_attn.k_proj": "colwise",
        "layers.*.self_attn.v_proj": "colwise",
        "layers.*.self_attn.o_proj": "rowwise",
        "layers.*.mlp.gate_proj": "colwise",
        "layers.*.mlp.up_proj": "colwise",
        "layers.*.mlp.down_proj": "rowwise",
    }
    base_model_pp_plan = {
        "embed_tokens": (["input_ids"], ["inputs_embeds"]),
        "layers": (["hidden_states", "attention_mask"], ["hidden_states"]),
        "norm": (["hidden_states"], ["hidden_states"]),
    }

    def __init__(self, vocab_size=152064, hidden_size=8192, intermediate_size=29568, num_hidden_layers=80,
                 num_attention_heads=64, num_key_value_heads=8, hidden_act="silu", max_position_embeddings=32768,
                 initializer_range=0.02, rms_norm_eps=1e-05, use_cache=True, tie_word_embeddings=False,
                 rope_theta=1000000.0, use_sliding_window=False, sliding_window=4096, max_window_layers=80,
                 attention_dropout=0.0, vision_config=None, rope_scaling=None, num_experts=4, experts=None,
                 dof_config=None, agent_pos_config=None, noise_scheduler=None, dim_inputs=(1536, 1536),
                 attention_moe=False, mlp_moe=False, image_token_id=151655, video_token_id=151656,
                 vision_start_token_id=151652, vision_end_token_id=151653, pad_token_id=None,
                 mrope_layout="hf", action_attn="bidirectional", **kwargs):
        if isinstance(vision_config, dict):
            self.vision_config = Qwen2_5_VLVisionConfig(**vision_config)
        elif vision_config is None:
            self.vision_config = Qwen2_5_VLVisionConfig()
        else:
            self.vision_config = vision_config
        self.vocab_size = vocab_size
        self.max_position_embeddings = max_position_embeddings
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.num_hidden_layers = num_hidden_layers
        self.num_attention_heads = num_attention_heads
        self.use_sliding_window = use_sliding_window
        self.sliding_window = sliding_window
        self.max_window_layers = max_window_layers
        self.num_key_value_heads = num_attention_heads if num_key_value_heads is None else num_key_value_heads
        self.hidden_act = hidden_act
        self.initializer_range = initializer_range
        self.rms_norm_eps = rms_norm_eps
        self.use_cache = use_cache
        self.tie_word_embeddings = tie_word_embeddings
        self.rope_theta = rope_theta
        self.attention_dropout = attention_dropout
        self.rope_scaling = copy.deepcopy(rope_scaling)
        self.num_experts = num_experts
        self.experts = copy.deepcopy(experts)
        self.dof_config = copy.deepcopy(dof_config)
        self.agent_pos_config = copy.deepcopy(agent_pos_config)
        self.noise_scheduler = copy.deepcopy(noise_scheduler) if noise_scheduler is not None else {}
        self.dim_inputs = tuple(dim_inputs)
        self.attention_moe = attention_moe
        self.mlp_moe = mlp_moe
        self.image_token_id = image_token_id
        self.video_token_id = video_token_id
        self.vision_start_token_id = vision_start_token_id
        self.vision_end_token_id = vision_end_token_id
        self.pad_token_id = pad_token_id
        # "hf": channel split t/h/w/t/h/w (valid rotation; what eager/sdpa use).
        # "wallx_cuda": contiguous 2x sections t,h,w (what the reference's CUDA rope kernel does).
        self.mrope_layout = mrope_layout
        # "bidirectional": action tokens attend to each other in both directions (4-D mask path).
        # "causal": pure causal, as the reference's flash-attention path.
        self.action_attn = action_attn
        if self.rope_scaling is not None and "type" in self.rope_scaling:
            if self.rope_scaling["type"] == "mrope":
                self.rope_scaling["type"] = "default"
            self.rope_scaling["rope_type"] = self.rope_scaling["type"]
        self.output_attentions = kwargs.pop("output_attentions", False)
        self.output_hidden_states = kwargs.pop("output_hidden_states", False)
        self.use_return_dict = kwargs.pop("use_return_dict", True)
        for k, v in kwargs.items():
            setattr(self, k, v)
        self.validate()

    # ------------------------------------------------------------------ helpers
    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def mrope_section(self) -> List[int]:
        if self.rope_scaling and "mrope_section" in self.rope_scaling:
            return list(self.rope_scaling["mrope_section"])
        half = self.head_dim // 2
        t = half // 4
        h = (half - t) // 2
        return [t, h, half - t - h]

    def expert_intermediate_sizes(self) -> List[int]:
        if not self.mlp_moe:
            return [self.intermediate_size]
        if not self.experts:
            raise ValueError("mlp_moe=True needs config.experts (a list of per-expert dicts)")
        return [int(e["intermediate_size"]) for e in self.experts[: self.num_experts]]

    def validate(self) -> None:
        if self.hidden_size % self.num_attention_heads:
            raise ValueError("hidden_size must be divisible by num_attention_heads")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
        if sum(self.mrope_section) != self.head_dim // 2:
            raise ValueError(f"mrope_section {self.mrope_section} must sum to head_dim/2 = {self.head_dim // 2}")
        if self.mrope_layout not in ("hf", "wallx_cuda"):
            raise ValueError("mrope_layout must be 'hf' or 'wallx_cuda'")
        if self.action_attn not in ("bidirectional", "causal"):
            raise ValueError("action_attn must be 'bidirectional' or 'causal'")
        if self.mlp_moe and self.experts is not None and len(self.experts) < self.num_experts:
            raise ValueError("config.experts has fewer entries than num_experts")

    # ------------------------------------------------------------------ I/O
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen2_5_VLConfig":
        d = dict(d)
        for drop in ("architectures", "transformers_version", "model_type", "torch_dtype", "dtype"):
            d.pop(drop, None)
        return cls(**d)

    @classmethod
    def from_pretrained(cls, path: str, **overrides) -> "Qwen2_5_VLConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
        d.update(overrides)
        return cls.from_dict(d)

    def to_dict(self) -> Dict[str, Any]:
        d = super().to_dict()
        d["dim_inputs"] = list(self.dim_inputs)
        d["model_type"] = self.model_type
        d["architectures"] = ["Qwen2_5_VLMoEForAction"]
        return d

    def save_pretrained(self, directory: str) -> None:
        os.makedirs(directory, exist_ok=True)
        with open(os.path.join(directory, "config.json"), "w", encoding="utf-8") as f:
            json.dump(self.to_dict(), f, indent=2)


def tiny_config(**overrides) -> Qwen2_5_VLConfig:
    """The 2-layer CPU correctness configuration (hidden 256, 4/2 heads, experts 512/256)."""
    base = dict(
        vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=4096,
        rope_scaling={"type": "mrope", "mrope_section": [8, 12, 12]},
        vision_config=dict(depth=2, hidden_size=128, intermediate_size=256, num_heads=4, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, window_size=112, out_hidden_size=256,
                           fullatt_block_indexes=[1]),
        num_experts=2, mlp_moe=True,
        experts=[dict(hidden_size=256, intermediate_size=512, hidden_act="silu"),
                 dict(hidden_size=256, intermediate_size=256, hidden_act="silu")],
        dof_config={"arm": 14}, agent_pos_config={"arm": 14}, noise_scheduler={"beta_alpha": 1.5, "beta_beta": 1.0, "s": 0.999},
        image_token_id=1001, video_token_id=1002, vision_start_token_id=1003, vision_end_token_id=1004, pad_token_id=0,
    )
    base.update(overrides)
    return Qwen2_5_VLConfig(**base)


def wall_oss_config(action_expert_intermediate: int = 2048, action_vocab: int = 2048, **overrides) -> Qwen2_5_VLConfig:
    """WALL-OSS-size configuration (Qwen2.5-VL-3B backbone + action expert).

    The action expert's FFN width is only in the released checkpoint's ``config.json``; it is a
    parameter here. Vocabulary = 151936 + 2 special tokens + the FAST action-token range.
    """
    base = dict(
        vocab_size=151936 + 2 + action_vocab, hidden_size=2048, intermediate_size=11008, num_hidden_layers=36,
        num_attention_heads=16, num_key_value_heads=2, rms_norm_eps=1e-6, rope_theta=1000000.0,
        max_position_embeddings=128000, rope_scaling={"type": "mrope", "mrope_section": [16, 24, 24]},
        vision_config=dict(depth=32, hidden_size=1280, intermediate_size=3420, num_heads=16, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, window_size=112, out_hidden_size=2048,
                           fullatt_block_indexes=[7, 15, 23, 31]),
        num_experts=2, mlp_moe=True,
        experts=[dict(hidden_size=2048, intermediate_size=11008, hidden_act="silu"),
                 dict(hidden_size=2048, intermediate_size=action_expert_intermediate, hidden_act="silu")],
        dof_config={"action": 20}, agent_pos_config={"proprio": 20},
        noise_scheduler={"beta_alpha": 1.5, "beta_beta": 1.0, "s": 0.999},
        image_token_id=151655, video_token_id=151656, vision_start_token_id=151652, vision_end_token_id=151653,
        pad_token_id=151643,
    )
    base.update(overrides)
    return Qwen2_5_VLConfig(**base)

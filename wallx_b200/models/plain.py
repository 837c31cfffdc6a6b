"""Plain Qwen2.5-VL (no expert routing, no action head in use): the base model of the VLA stack.

The reference ships the whole Hugging Face Qwen2.5-VL family next to its VLA model
(wall_x/model/qwen2_5_based/modeling_qwen2_5_vl.py: ``Qwen2_5_VLModel`` :1231,
``Qwen2_5_VLForConditionalGeneration`` :1685, the vision tower :438, ``Qwen2_5_VLDecoderLayer``
:1132, ``Qwen2MLP`` :715). Here the same kernels and modules serve both: a decoder layer runs a
single SwiGLU FFN when ``config.mlp_moe`` is off, so the plain model is the VLA class with that
switch forced and every token treated as a VLM token. Checkpoints in the Hugging Face key layout
(``model.layers.N.mlp.gate_proj.weight`` ...) load directly.
"""
from __future__ import annotations

from ..config import Qwen2_5_VLConfig
from .layers import RMSNorm, SwiGLUFFN
from .llm import Attention, DecoderLayer, Qwen2_5_VLMoEModel
from .rotary import (Qwen2_5_VisionRotaryEmbedding, Qwen2_5_VLRotaryEmbedding, apply_multimodal_rotary_pos_emb,  # noqa: F401
                     apply_rotary_pos_emb_flashatt, apply_rotary_pos_emb_vision, repeat_kv, rotate_half)
from .vision import PatchMerger, VisionAttention, VisionBlock, VisionPatchEmbed, VisionTransformer
from .vla import Qwen2_5_VLACausalLMOutputWithPast, Qwen2_5_VLMoEForAction


class Qwen2_5_VLForConditionalGeneration(Qwen2_5_VLMoEForAction):
    """Vision-language model for text training (next-token cross entropy) and generation."""

    def __init__(self, config: Qwen2_5_VLConfig, processor=None, **kwargs):
        config.mlp_moe = False
        config.num_experts = max(1, int(getattr(config, "num_experts", 1) or 1))
        if not getattr(config, "dof_config", None):
            config.dof_config = {"unused": 8}
        if not getattr(config, "agent_pos_config", None):
            config.agent_pos_config = {"unused": 8}
        super().__init__(config, processor=processor, **kwargs)


class Qwen2_5_VLModel(Qwen2_5_VLMoEModel):
    """Embedding + decoder stack + final norm with one FFN per layer."""

    def __init__(self, config: Qwen2_5_VLConfig):
        config.mlp_moe = False
        super().__init__(config)


# names of the reference's building blocks
Qwen2_5_VisionTransformerPretrainedModel = VisionTransformer
Qwen2_5_VisionPatchEmbed = VisionPatchEmbed
Qwen2_5_VLVisionBlock = VisionBlock
Qwen2_5_VLPatchMerger = PatchMerger
Qwen2_5_VLDecoderLayer = DecoderLayer
Qwen2RMSNorm = RMSNorm
Qwen2MLP = SwiGLUFFN
Qwen2_5_VLMLP = SwiGLUFFN
Qwen2_5_VLCausalLMOutputWithPast = Qwen2_5_VLACausalLMOutputWithPast
Qwen2_5_VLPreTrainedModel = Qwen2_5_VLMoEForAction  # from_pretrained / save_pretrained / state-dict hooks live there
# One attention implementation per tower: the reference's eager / flash-attn 2 / SDPA variants are all
# served by the same tcgen05 attention kernels, whatever ``attn_implementation`` a config names.
Qwen2_5_VLAttention = Qwen2_5_VLFlashAttention2 = Qwen2_5_VLSdpaAttention = Attention
QWEN2_5_VL_ATTENTION_CLASSES = {"eager": Attention, "flash_attention_2": Attention, "sdpa": Attention}
Qwen2_5_VLVisionAttention = Qwen2_5_VLVisionFlashAttention2 = Qwen2_5_VLVisionSdpaAttention = VisionAttention
QWEN2_5_VL_VISION_ATTENTION_CLASSES = {"eager": VisionAttention, "flash_attention_2": VisionAttention, "sdpa": VisionAttention}

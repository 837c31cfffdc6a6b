"""The reference's plain Qwen2.5-VL module path; every name resolves to this framework's modules."""
from wallx_b200.models.plain import (QWEN2_5_VL_ATTENTION_CLASSES, QWEN2_5_VL_VISION_ATTENTION_CLASSES,  # noqa: F401
                                     Qwen2_5_VisionPatchEmbed, Qwen2_5_VisionRotaryEmbedding,
                                     Qwen2_5_VisionTransformerPretrainedModel, Qwen2_5_VLAttention,
                                     Qwen2_5_VLCausalLMOutputWithPast, Qwen2_5_VLDecoderLayer, Qwen2_5_VLFlashAttention2,
                                     Qwen2_5_VLForConditionalGeneration, Qwen2_5_VLMLP, Qwen2_5_VLModel,
                                     Qwen2_5_VLPatchMerger, Qwen2_5_VLPreTrainedModel, Qwen2_5_VLRotaryEmbedding,
                                     Qwen2_5_VLSdpaAttention, Qwen2_5_VLVisionAttention, Qwen2_5_VLVisionBlock,
                                     Qwen2_5_VLVisionFlashAttention2, Qwen2_5_VLVisionSdpaAttention, Qwen2MLP,
                                     Qwen2RMSNorm, apply_multimodal_rotary_pos_emb, apply_rotary_pos_emb_flashatt,
                                     apply_rotary_pos_emb_vision, repeat_kv, rotate_half)

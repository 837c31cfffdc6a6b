from wallx_b200.models.plain import (Qwen2_5_VisionPatchEmbed, Qwen2_5_VisionTransformerPretrainedModel,  # noqa: F401
                                     Qwen2_5_VLCausalLMOutputWithPast, Qwen2_5_VLDecoderLayer,
                                     Qwen2_5_VLForConditionalGeneration, Qwen2_5_VLMLP, Qwen2_5_VLModel,
                                     Qwen2_5_VLPatchMerger, Qwen2_5_VLVisionBlock, Qwen2MLP, Qwen2RMSNorm)

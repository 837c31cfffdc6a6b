from ..config import Qwen2_5_VLConfig, Qwen2_5_VLVisionConfig
from .llm import Qwen2_5_VLMoEModel
from .vla import Qwen2_5_VLACausalLMOutputWithPast, Qwen2_5_VLMoEForAction
from .plain import Qwen2_5_VLForConditionalGeneration, Qwen2_5_VLModel

__all__ = ["Qwen2_5_VLConfig", "Qwen2_5_VLVisionConfig", "Qwen2_5_VLMoEModel", "Qwen2_5_VLMoEForAction",
           "Qwen2_5_VLACausalLMOutputWithPast", "Qwen2_5_VLForConditionalGeneration", "Qwen2_5_VLModel"]

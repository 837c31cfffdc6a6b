from wallx_b200.config import Qwen2_5_VLConfig  # noqa: F401
from wallx_b200.models import Qwen2_5_VLMoEForAction, Qwen2_5_VLMoEModel  # noqa: F401

__all__ = ["Qwen2_5_VLConfig", "Qwen2_5_VLMoEModel", "Qwen2_5_VLMoEForAction"]

from wallx_b200.models.vla import Qwen2_5_VLACausalLMOutputWithPast, Qwen2_5_VLMoEForAction  # noqa: F401
from wallx_b200.models.llm import Qwen2_5_VLMoEModel  # noqa: F401

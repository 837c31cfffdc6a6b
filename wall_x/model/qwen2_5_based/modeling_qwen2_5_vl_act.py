"""The reference's VLA module path; every name resolves to this framework's modules."""
from wallx_b200.models.layers import SwiGLUFFN as BlockSparseMLP  # noqa: F401  one SwiGLU expert
from wallx_b200.models.llm import DecoderLayer as Qwen2_5_VLDecoderLayer_with_MoE  # noqa: F401
from wallx_b200.models.llm import Qwen2_5_VLMoEModel, SparseMoeBlock  # noqa: F401
from wallx_b200.models.plain import QWEN2_5_VL_ATTENTION_CLASSES  # noqa: F401
from wallx_b200.models.vla import Qwen2_5_VLACausalLMOutputWithPast, Qwen2_5_VLMoEForAction  # noqa: F401

from wallx_b200.config import Qwen2_5_VLConfig, Qwen2_5_VLVisionConfig  # noqa: F401

from wallx_b200.data.config import *  # noqa: F401,F403
from wallx_b200.data.config import ACTION_DATASET_NAMES, MULTIMODAL_DATASET_NAMES, X2RDataProcessingConfig  # noqa: F401

from wallx_b200.data.config import MULTIMODAL_DATASET_NAMES  # noqa: F401
from wallx_b200.data.text import (CAMERA_NAME_MAPPING, FREQUENCY_MAPPING, get_action_tokens, get_frame_instruction,  # noqa: F401
                                  get_task_instruction, get_wallx_normal_text, pad_action_token_strs,
                                  preprocesser_call, process_grounding_points, replace_action_token)

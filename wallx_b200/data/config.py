"""Data-side configuration: dataset name registries and the typed processing config.

Same names and defaults as the reference's ``wall_x/data/config.py:7-124``; the Qwen image-size
constants it takes from ``qwen_vl_utils`` (not installed here) are restated.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

IMAGE_FACTOR = 28
MIN_PIXELS = 4 * 28 * 28
MAX_PIXELS = 16384 * 28 * 28

TACTILE_FILE_MAPPING = {"tactile_data_left": "left_tactile", "tactile_data_right": "right_tactile"}

ACTION_DATASET_NAMES: List[str] = (
    "x2_normal agibotworld_alpha droid fractal bridge_data_v2 DobbE RH20T UMI-biarm austin_buds austin_sailor "
    "austin_sirius bc_z berkeley_autolab_ur5 berkeley_cable_routing berkeley_fanuc_manipulation "
    "dlr_edan_shared_control fmb furniture_bench jaco_play nyu_rot stanford_hydra stanford_kuka_multimodal "
    "taco_play utaustin_mutex viola"
).split()

MULTIMODAL_DATASET_NAMES: List[str] = (
    "x2_multimodal_from_action x2_multimodal x2_subtask_generation multimodal_CapsFusion multimodal_Robo2VLM "
    "multimodal_RoboPoint multimodal_EQA multimodal_Cambrian multimodal_pixmo multimodal_VQAv2 multimodal_COCO"
).split()


@dataclass
class X2RDataProcessingConfig:
    predict_action_keys: List[str] = field(default_factory=list)
    obs_action_keys: List[str] = field(default_factory=list)
    resolution: Dict[str, int] = field(
        default_factory=lambda: {"face_view": -1, "left_wrist_view": 128, "right_wrist_view": 128})
    train_test_split: float = 0.9
    split_seed: int = 42
    priority_order: Optional[Dict[str, float]] = None
    model_type: str = "qwen2_5"
    max_pixels: int = MAX_PIXELS
    min_pixels: int = MIN_PIXELS
    image_factor: int = IMAGE_FACTOR
    generate_subtask_ratio: float = 0.0

    def __post_init__(self):
        if not 0 < self.train_test_split < 1:
            raise ValueError(f"train_test_split must be between 0 and 1, got {self.train_test_split}")

    def as_dict(self) -> Dict:
        return self.__dict__

    def update(self, **kwargs) -> "X2RDataProcessingConfig":
        for key, value in kwargs.items():
            if not hasattr(self, key):
                raise ValueError(f"Unknown configuration parameter: {key}")
            setattr(self, key, value)
        return self

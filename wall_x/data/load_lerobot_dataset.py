from wallx_b200.data.collator import DataCollator  # noqa: F401
from wallx_b200.data.lerobot import (CAMERA_KEY_MAPPINGS, PreprocessedDataset, TestDataset, get_data_configs,  # noqa: F401
                                     get_distributed_dataloader, load_lerobot_data, load_test_dataset)

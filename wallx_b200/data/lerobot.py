"""LeRobot-style datasets -> samples for :class:`DataCollator`.

Mirrors ``wall_x/data/load_lerobot_dataset.py``: ``PreprocessedDataset`` (95/5 random split,
per-camera aspect-preserving resize to ``resolution[cam]`` then rounding to multiples of 28 px,
prompt text, grounding-point rescale) (:43-236), ``load_lerobot_data`` (action chunks through
``delta_timestamps``) (:418-514), ``get_data_configs`` (defaults; ``action_horizon += 1``)
(:541-561), ``TestDataset`` / ``load_test_dataset`` (:564-637) and ``CAMERA_KEY_MAPPINGS`` (:23-29).
The ``lerobot`` package is only needed by :func:`load_lerobot_data`; everything else works with any
dataset object that offers ``__getitem__``, ``__len__`` and a ``meta`` with ``repo_id``,
``camera_keys`` and ``stats`` -- :class:`SyntheticEpisodeDataset` is such an object.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
from torch.utils.data import DataLoader, DistributedSampler, random_split

from .collator import DataCollator
from .config import X2RDataProcessingConfig
from .synthetic import smart_resize
from .text import get_wallx_normal_text, process_grounding_points

CAMERA_KEY_MAPPINGS = {
    "lerobot/aloha_mobile_cabinet": {
        "observation.images.cam_high": "face_view",
        "observation.images.cam_left_wrist": "left_wrist_view",
        "observation.images.cam_right_wrist": "right_wrist_view",
    },
    "synthetic/episodes": {
        "observation.images.cam_high": "face_view",
        "observation.images.cam_left_wrist": "left_wrist_view",
        "observation.images.cam_right_wrist": "right_wrist_view",
    },
}


def get_data_configs(config: Dict) -> Dict:
    """Fill data defaults the way the reference does; the chunk is one step longer than the horizon."""
    out = dict(config)
    out.setdefault("train_test_split", 0.95)
    out.setdefault("split_seed", 42)
    out.setdefault("action_horizon", 32)
    out.setdefault("predict_action_keys", [])
    out.setdefault("obs_action_keys", [])
    out.setdefault("resolution", None)
    out.setdefault("priority_order", None)
    out["action_horizon"] = int(out["action_horizon"]) + 1
    return out


class _Meta:
    def __init__(self, repo_id, camera_keys, stats):
        self.repo_id, self.camera_keys, self.stats = repo_id, camera_keys, stats


class SyntheticEpisodeDataset:
    """Random frames/actions with the LeRobot sample layout (float CHW images in [0, 1])."""

    def __init__(self, n: int = 64, image_hw=(96, 128), action_dim: int = 14, horizon: int = 32, seed: int = 0,
                 repo_id: str = "synthetic/episodes"):
        g = torch.Generator().manual_seed(seed)
        self.n, self.hw, self.horizon = n, image_hw, horizon
        self.actions = torch.randn((n, horizon, action_dim), generator=g)
        self.states = torch.randn((n, action_dim), generator=g)
        self.seed = seed
        cams = list(CAMERA_KEY_MAPPINGS[repo_id].keys())
        import numpy as np

        self.meta = _Meta(repo_id, cams, {"action": {"min": np.full((action_dim,), -3.0, dtype="float32"),
                                                    "max": np.full((action_dim,), 3.0, dtype="float32")}})

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 100003 + int(i))
        item = {k: torch.rand((3, self.hw[0], self.hw[1]), generator=g) for k in self.meta.camera_keys}
        item["action"] = self.actions[i]
        item["observation.state"] = self.states[i]
        item["frame_index"] = torch.tensor(int(i))
        item["task"] = "pick up the object and place it in the bin"
        return item


class PreprocessedDataset:
    def __init__(self, dataset, config: Dict, dataload_config: Dict, seed: Optional[int] = 42, rank: int = 0,
                 world_size: int = 1, test_only: bool = False, processor=None, action_tokenizer=None, model_config=None):
        self.hf_dataset = dataset
        self.config, self.dataload_config = config, dataload_config
        self.seed, self.rank, self.world_size = seed, rank, world_size
        self.processor, self.action_tokenizer, self.model_config = processor, action_tokenizer, model_config
        if test_only:
            self._dataset = dataset
            self.train_dataset = self.val_dataset = dataset
        else:
            gen = torch.Generator().manual_seed(seed) if seed is not None else None
            self.train_dataset, self.val_dataset = random_split(dataset, [0.95, 0.05], gen)
            self._dataset = self.train_dataset
        self.use_fast_tokenizer = bool(config.get("use_fast_tokenizer", False))
        self.data_config = X2RDataProcessingConfig().update(
            train_test_split=dataload_config.get("train_test_split", 0.95),
            split_seed=dataload_config.get("split_seed", 42),
            predict_action_keys=dataload_config.get("predict_action_keys", []),
            obs_action_keys=dataload_config.get("obs_action_keys", []),
            resolution=dataload_config.get("resolution") or {},
            priority_order=dataload_config.get("priority_order"))
        self._cam_key_mapping = CAMERA_KEY_MAPPINGS[dataset.meta.repo_id]
        self.chunk = int(dataload_config.get("action_horizon", 33)) - 1

    def _vision_preprocess(self, frames):
        from PIL import Image

        out = []
        oh = ow = rh = rw = 0
        for key in self.hf_dataset.meta.camera_keys:
            img = Image.fromarray((frames[key].permute(1, 2, 0) * 255).to(torch.uint8).cpu().numpy())
            ow, oh = img.size
            target = self.data_config.resolution.get(self._cam_key_mapping[key], -1)
            if target != -1:
                if ow > oh:
                    img = img.resize((target, int(target * oh / ow)))
                else:
                    img = img.resize((int(target * ow / oh), target))
            cw, ch = img.size
            rh, rw = smart_resize(ch, cw, factor=self.data_config.image_factor, min_pixels=self.data_config.min_pixels,
                                  max_pixels=self.data_config.max_pixels)
            out.append(img.resize((rw, rh)))
        return out, oh, ow, rh, rw

    def __getitem__(self, index):
        data = self._dataset[index]
        images, h, w, rh, rw = self._vision_preprocess(data)
        text, _ = get_wallx_normal_text({"instruction": data["task"]}, self.chunk, int(data["frame_index"]),
                                        self.data_config.priority_order, self._cam_key_mapping,
                                        generate_subtask_ratio=self.data_config.generate_subtask_ratio)
        text = process_grounding_points(text, h, w, rh, rw, self.data_config.model_type)
        return {"image_inputs": images, "text": text, "action": data["action"], "agent_pos": data["observation.state"],
                "frame_index": data["frame_index"]}

    def __len__(self):
        return len(self._dataset)

    def _eval(self):
        self._dataset = self.val_dataset

    def _train(self):
        self._dataset = self.train_dataset

    def _collator(self):
        return DataCollator(self.config, self.dataload_config, self.hf_dataset.meta.stats, processor=self.processor,
                            action_tokenizer=self.action_tokenizer, model_config=self.model_config)

    def _loader(self, train: bool):
        bs = self.config.get("batch_size_per_gpu", 8) if train else self.config.get(
            "eval_batch_size_per_gpu", self.config.get("batch_size_per_gpu", 8))
        workers = self.config.get("num_workers", 4)
        sampler = DistributedSampler(self, num_replicas=self.world_size, rank=self.rank, shuffle=train,
                                     seed=self.seed if self.seed is not None else 0, drop_last=train)
        kw = dict(prefetch_factor=2, persistent_workers=True) if workers > 0 else {}
        loader = DataLoader(self, batch_size=bs, sampler=sampler, num_workers=workers, collate_fn=self._collator(),
                            pin_memory=torch.cuda.is_available(), drop_last=train, **kw)
        return loader, sampler

    def get_train_dataloader(self):
        self._train()
        return self._loader(True)

    def get_val_dataloader(self):
        self._eval()
        return self._loader(False)


def get_distributed_dataloader(dataset, config=None, rank: int = 0, world_size: int = 1, seed: int = 42, is_train: bool = True):
    """``(loader, sampler)`` of a :class:`PreprocessedDataset` for one rank (load_lerobot_dataset.py:517-538).
    ``config`` is accepted for signature parity; the dataset already holds it."""
    dataset.rank, dataset.world_size = int(rank), int(world_size)
    if is_train:
        dataset.seed = seed
        return dataset.get_train_dataloader()
    return dataset.get_val_dataloader()


def load_lerobot_data(config: Dict, lerobot_config: Dict, rank: int = 0, world_size: int = 1, seed: int = 42,
                      processor=None, action_tokenizer=None, model_config=None) -> PreprocessedDataset:
    """Open a LeRobot dataset with an action chunk of ``action_horizon - 1`` future steps."""
    try:
        from lerobot.datasets.lerobot_dataset import LeRobotDataset, LeRobotDatasetMetadata
    except Exception as e:  # pragma: no cover - lerobot is not part of this image
        raise ImportError("load_lerobot_data needs the `lerobot` package") from e
    dataload_config = get_data_configs(config["data"])
    repo_id = lerobot_config.get("repo_id")
    meta = LeRobotDatasetMetadata(repo_id, root=lerobot_config.get("root"))
    horizon = dataload_config["action_horizon"] - 1
    delta = {"action": [t / meta.fps for t in range(horizon)]}
    kwargs = {k: lerobot_config.get(k) for k in ("root", "episodes", "image_transforms", "revision", "video_backend")}
    ds = LeRobotDataset(repo_id, delta_timestamps=lerobot_config.get("delta_timestamps") or delta,
                        tolerance_s=lerobot_config.get("tolerance_s", 1e-4),
                        force_cache_sync=lerobot_config.get("force_cache_sync", False),
                        download_videos=lerobot_config.get("download_videos", True), **kwargs)
    return PreprocessedDataset(ds, config, dataload_config, seed=seed, rank=rank, world_size=world_size,
                               processor=processor, action_tokenizer=action_tokenizer, model_config=model_config)


class TestDataset(PreprocessedDataset):
    """Whole dataset, no split (open-loop evaluation)."""

    __test__ = False  # not a pytest class

    def __init__(self, dataset, config, dataload_config, **kw):
        super().__init__(dataset, config, dataload_config, test_only=True, **kw)

    def get_dataloader(self):
        """Frames in order, batch size 1, no shuffling (reference: load_lerobot_dataset.py:564-620)."""
        return DataLoader(self, batch_size=1, shuffle=False, num_workers=0, collate_fn=self._collator())


def load_test_dataset(config: Dict, lerobot_config: Dict, seed: int = 42, dataset=None, **kw):
    dataload_config = get_data_configs(config["data"])
    if dataset is None:
        pre = load_lerobot_data(config, lerobot_config, seed=seed, **kw)
        dataset = pre.hf_dataset
    return TestDataset(dataset, config, dataload_config, seed=seed, **kw)

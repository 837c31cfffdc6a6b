"""Host-side batch finishing: packing info, position ids and label rows computed on the CPU.

The collator already holds every index-like quantity on the host (ids, masks, grids), so the
things the reference computes on the device with host round-trips (expert counts,
modeling_qwen2_5_vl_act.py:1275-1283; ViT seqlens ``.item()``s, modeling_qwen2_5_vl.py:600-603) are
attached to the batch here and travel with it. The model falls back to computing them itself
(with a sync) when a batch comes without them.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import ref


def add_pack_info(batch: Dict[str, object], config, with_positions: bool = True) -> Dict[str, object]:
    ids: torch.Tensor = batch["input_ids"]
    B, S = ids.shape
    am = batch.get("attention_mask")
    if am is None:
        am = torch.ones_like(ids)
    amb = am.to(torch.bool)
    batch["seq_lens"] = amb.sum(1).to(torch.int64)
    batch["pack_index"] = torch.nonzero(amb.reshape(-1), as_tuple=False).squeeze(1)
    grid = batch.get("image_grid_thw")
    if grid is not None:
        batch["image_grid_host"] = [[int(v) for v in row] for row in grid.tolist()]
    vgrid = batch.get("video_grid_thw")
    if vgrid is not None:
        batch["video_grid_host"] = [[int(v) for v in row] for row in vgrid.tolist()]
    if with_positions and "position_ids" not in batch:
        vc = config.vision_config
        pos, _ = ref.rope_index(ids, grid, vgrid, batch.get("second_per_grid_ts"), am, vc.spatial_merge_size,
                                config.image_token_id, config.video_token_id, config.vision_start_token_id,
                                vc.tokens_per_second)
        batch["position_ids"] = pos
    labels = batch.get("labels")
    if labels is not None:
        shift = torch.cat([labels[:, 1:], labels.new_full((B, 1), -100)], dim=1).reshape(-1)
        shift = shift.index_select(0, batch["pack_index"])
        cu = torch.cumsum(batch["seq_lens"], 0)
        shift[cu - 1] = -100
        batch["label_index"] = torch.nonzero(shift != -100, as_tuple=False).squeeze(1)
    return batch


def to_device(batch: Dict[str, object], device, dtype=None, non_blocking: bool = True) -> Dict[str, object]:
    """Move tensors to ``device`` (floating tensors to ``dtype``); lists and host tables stay."""
    host_keys = {"seq_lens", "image_grid_host", "video_grid_host", "dataset_names"}
    out = {}
    for k, v in batch.items():
        if isinstance(v, torch.Tensor) and k not in host_keys:
            if v.is_floating_point() and dtype is not None:
                out[k] = v.to(device=device, dtype=dtype, non_blocking=non_blocking)
            else:
                out[k] = v.to(device=device, non_blocking=non_blocking)
        else:
            out[k] = v
    return out


def pin_batch(batch: Dict[str, object]) -> Dict[str, object]:
    return {k: (v.pin_memory() if isinstance(v, torch.Tensor) and not v.is_pinned() else v) for k, v in batch.items()}


# ------------------------------------------------------------------------------------ DataCollator
ACTION_PAD_DIM = 20  # actions and proprio are zero-padded to 20 dims (load_lerobot_dataset.py:317,349)


def minmax_normalize(x: torch.Tensor, min_stat, max_stat) -> torch.Tensor:
    """``(x - min) / delta * 2 - 1`` clamped to [-1, 1]; a zero range counts as 1."""
    mn = torch.as_tensor(min_stat, dtype=x.dtype)
    delta = torch.as_tensor(max_stat, dtype=x.dtype) - mn
    delta = torch.where(delta == 0, torch.ones_like(delta), delta)
    return torch.clamp((x - mn) / delta * 2 - 1, -1, 1)


def _pad_last(x: torch.Tensor, width: int) -> torch.Tensor:
    if x.shape[-1] >= width:
        return x
    return torch.cat([x, x.new_zeros(x.shape[:-1] + (width - x.shape[-1],))], dim=-1)


class DataCollator:
    """List of samples ``{image_inputs, text, action, agent_pos, frame_index}`` -> model batch.

    Follows the reference collator (load_lerobot_dataset.py:239-415): NaN entries become mask 0,
    min-max normalisation with the dataset statistics, zero-padding to 20 dims, FAST token
    substitution (or removal of the FAST slot in flow mode), placeholder expansion + tokenisation +
    assistant labels, ``moe_token_types = (input_ids == <|action|>)``, ``dataset_names``.
    On top of that the batch gets its host-side packing info (:func:`add_pack_info`).
    """

    def __init__(self, config: Dict, dataload_config: Dict, stats: Dict, processor=None, action_tokenizer=None,
                 model_config=None):
        from . import text as T

        self.T = T
        self.config = config
        self.dataload_config = dataload_config
        self.min_stat = stats["action"]["min"]
        self.max_stat = stats["action"]["max"]
        self.use_fast_tokenizer = bool(config.get("use_fast_tokenizer", False))
        self.processor, action_tokenizer = self.load_processor(processor, action_tokenizer)
        self.train_action_tokenizer = action_tokenizer if self.use_fast_tokenizer else None
        self.action_mapper = None
        if self.train_action_tokenizer is not None:
            tok = self.processor.tokenizer
            self.action_mapper = {tok.convert_tokens_to_ids(f"<|action_token_{i}|>"): i
                                  for i in range(self.train_action_tokenizer.vocab_size)}
        self.model_config = model_config
        self.max_length = dataload_config.get("max_length", 768)

    def _vector(self, items, key):
        x = torch.stack([torch.as_tensor(it[key], dtype=torch.float32) for it in items])
        if x.dim() == 2:
            x = x.unsqueeze(1)
        mask = (~torch.isnan(x)).float()
        x = minmax_normalize(torch.nan_to_num(x, nan=0.0), self.min_stat, self.max_stat)
        return _pad_last(x, ACTION_PAD_DIM), _pad_last(mask, ACTION_PAD_DIM)

    _processor_cache: Dict[str, object] = {}  # one processor per path and process (DataLoader workers re-create collators)

    def load_processor(self, processor=None, action_tokenizer=None):
        """``(processor, action_tokenizer)``: the given objects, else loaded from ``pretrained_wallx_path`` /
        ``action_tokenizer_path`` (cached per path), else -- FAST branch without a tokenizer path -- the built-in DCT
        tokenizer over the checkpoint's action id range (reference: load_lerobot_dataset.py:254-285)."""
        config = self.config
        if processor is None:
            path = config["pretrained_wallx_path"]
            if path not in DataCollator._processor_cache:
                from transformers import AutoProcessor

                DataCollator._processor_cache[path] = AutoProcessor.from_pretrained(path, use_fast=True)
            processor = DataCollator._processor_cache[path]
        if config.get("padding_side", "left") == "left":
            processor.tokenizer.padding_side = "left"
        if self.use_fast_tokenizer and action_tokenizer is None:
            action_tokenizer = getattr(processor, "action_processor", None)
        if self.use_fast_tokenizer and action_tokenizer is None:
            path = config.get("action_tokenizer_path")
            if path:
                if path not in DataCollator._processor_cache:
                    from transformers import AutoProcessor

                    DataCollator._processor_cache[path] = AutoProcessor.from_pretrained(path, trust_remote_code=True)
                action_tokenizer = DataCollator._processor_cache[path]
            else:
                from .fast_tokenizer import DctActionTokenizer

                action_tokenizer = DctActionTokenizer(int(processor.tokenizer.init_kwargs["action_token_vocab_size"]))
        return processor, action_tokenizer

    @classmethod
    def _normalize(cls, action: torch.Tensor, min_stat, delta) -> torch.Tensor:
        """Min-max normalisation from ``min`` and ``delta = max - min`` (reference: load_lerobot_dataset.py:294-304)."""
        mn = torch.as_tensor(min_stat, dtype=action.dtype)
        return minmax_normalize(action, mn, mn + torch.as_tensor(delta, dtype=action.dtype))

    def __call__(self, items):
        known = {"agent_pos", "action", "image_inputs", "text", "frame_index"}
        for k in items[0].keys():
            if k not in known:
                raise NotImplementedError(f"{k} input not implemented in preprocesser")
        out: Dict[str, object] = {}
        if "agent_pos" in items[0]:
            out["proprioception"], out["agent_pos_mask"] = self._vector(items, "agent_pos")
        if "action" in items[0]:
            out["action_chunk"], out["dof_mask"] = self._vector(items, "action")
        if "frame_index" in items[0]:
            out["frame_index"] = torch.stack([torch.as_tensor(it["frame_index"]) for it in items])
        names = ["x2_normal"] * len(items)
        text = self.T.replace_action_token([it["text"] for it in items], out.get("action_chunk"),
                                           self.train_action_tokenizer, names, out.get("dof_mask"))
        images = [im for it in items for im in it["image_inputs"]]
        enc = self.T.preprocesser_call(self.processor, images=images, text=text, videos=None, padding=True,
                                       truncation=True, max_length=self.max_length, return_tensors="pt")
        out.update(enc)
        action_id = self.processor.tokenizer.convert_tokens_to_ids("<|action|>")
        out["moe_token_types"] = out["input_ids"] == action_id
        out["dataset_names"] = names
        if out.get("labels") is None:
            out.pop("labels", None)
        if self.model_config is not None:
            add_pack_info(out, self.model_config)
        return out

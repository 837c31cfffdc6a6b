"""Host-side batch finishing: packing info, position ids and label rows computed on the CPU.

The collator already holds every index-like quantity on the host (ids, masks, grids), so the
things the reference computes on the device with host round-trips (expert counts,
modeling_qwen2_5_vl_act.py:1275-1283; ViT seqlens ``.item()``s, modeling_qwen2_5_vl.py:600-603) are
attached to the batch here and travel with it. The model falls back to computing them itself
(with a sync) when a batch comes without them.
"""
from __future__ import annotations

from typing import Dict, Optional

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

"""Index-generation operators: LLM 3-axis rope positions, ViT rotary ids and window permutation.

Public signatures mirror the reference's wrappers (wall_x/fusions/ops.py:507-742). Inputs that live
on the host (grid tables from the collator) are processed on the host with no device round trip;
CUDA inputs run the single-launch kernels of the extension.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from . import ref
from . import _ext


def _grid_list(grid_thw) -> List[List[int]]:
    if isinstance(grid_thw, torch.Tensor):
        return [[int(v) for v in row] for row in grid_thw.tolist()]
    return [[int(v) for v in row] for row in grid_thw]


def rot_pos_emb(inv_freq: torch.Tensor, grid_thw, spatial_merge_size: int) -> torch.Tensor:
    """ViT rotary angle table ``[sum(t*h*w), 2*len(inv_freq)]`` (csrc/rot_pos.cu:315-332)."""
    if isinstance(grid_thw, torch.Tensor) and grid_thw.is_cuda:
        return _ext.get().vit_rot_pos(inv_freq.float().contiguous(), grid_thw.to(torch.int32).contiguous(),
                                      int(spatial_merge_size), _total_patches(grid_thw))
    return ref.rot_pos_emb(inv_freq, _grid_list(grid_thw), spatial_merge_size)


def _total_patches(grid_thw: torch.Tensor) -> int:
    return int((grid_thw[:, 0] * grid_thw[:, 1] * grid_thw[:, 2]).sum().item())


def window_index(grid_thw, window_size: int, spatial_merge_size: int, patch_size: int):
    """``(window_index [sum t*h/m*w/m], cu_window_seqlens list)`` (csrc/window_index.cu:208-286)."""
    return ref.window_index(_grid_list(grid_thw), window_size, spatial_merge_size, patch_size)


def get_window_index(grid_thw, window_size: int, spatial_merge_size: int, patch_size: int, spatial_merge_unit: int = 4):
    """Reference-compatible name and return types (tensor index, tensor cu_seqlens)."""
    dev = grid_thw.device if isinstance(grid_thw, torch.Tensor) else "cpu"
    if isinstance(grid_thw, torch.Tensor) and grid_thw.is_cuda:
        grid = grid_thw.to(torch.int32).contiguous()
        n_merged, n_windows = _window_counts(_grid_list(grid_thw), window_size, spatial_merge_size, patch_size)
        return _ext.get().vit_window_index(grid, int(window_size // spatial_merge_size // patch_size),
                                           int(spatial_merge_size), int(n_merged), int(n_windows))
    idx, cu = window_index(grid_thw, window_size, spatial_merge_size, patch_size)
    return idx.to(dev), torch.tensor(cu, dtype=torch.int32, device=dev)


def _window_counts(grid: Sequence[Sequence[int]], window_size: int, merge: int, patch: int) -> Tuple[int, int]:
    vw = window_size // merge // patch
    n_merged = n_windows = 0
    for t, h, w in grid:
        gh, gw = h // merge, w // merge
        nh = (gh + vw - gh % vw) // vw
        nw = (gw + vw - gw % vw) // vw
        n_merged += t * gh * gw
        n_windows += t * nh * nw
    return n_merged, n_windows


def get_rope_index(input_ids: torch.Tensor, image_grid_thw=None, video_grid_thw=None, second_per_grid_ts=None,
                   attention_mask=None, spatial_merge_size: int = 2, image_token_id: int = 151655,
                   video_token_id: int = 151656, vision_start_token_id: int = 151652, tokens_per_second: float = 2.0):
    """``position_ids [3, B, S]`` and ``mrope_deltas [B, 1]`` (csrc/rope_index.cu:464-569 and the
    Python original modeling_qwen2_5_vl_act.py:929-1149)."""
    if input_ids.is_cuda and (image_grid_thw is not None or video_grid_thw is not None):
        C = _ext.get()
        dev = input_ids.device
        empty = torch.zeros((0, 3), dtype=torch.int32, device=dev)
        ig = image_grid_thw.to(device=dev, dtype=torch.int32).contiguous() if image_grid_thw is not None else empty
        vg = video_grid_thw.to(device=dev, dtype=torch.int32).contiguous() if video_grid_thw is not None else empty
        if second_per_grid_ts is not None:
            spg = second_per_grid_ts.to(device=dev, dtype=torch.float32).contiguous()
        else:
            spg = torch.ones((vg.shape[0],), dtype=torch.float32, device=dev)
        am = attention_mask.to(torch.int32).contiguous() if attention_mask is not None else None
        return C.rope_index(input_ids.contiguous(), am, ig, vg, spg, int(spatial_merge_size), int(image_token_id),
                            int(video_token_id), int(vision_start_token_id), float(tokens_per_second))
    return ref.rope_index(input_ids, image_grid_thw, video_grid_thw, second_per_grid_ts, attention_mask,
                          spatial_merge_size, image_token_id, video_token_id, vision_start_token_id, tokens_per_second)

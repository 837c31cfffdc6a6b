"""Generation plumbing and the dense attention-mask rule under the reference's method names.

This framework decodes with its own loop (``models/inference.py``: prefix pass into a KV cache, one-token steps,
interval tables instead of dense masks), so nothing here is on a hot path. The functions exist for user code that
drives the model through the Hugging Face generation hooks, and as the dense oracle of the attention rule:

* :func:`dense_attention_mask` / ``Qwen2_5_VLMoEModel._update_causal_mask`` /
  ``_prepare_4d_causal_attention_mask_with_cache_position``: additive ``[B, 1, Q, K]`` mask, causal by cache
  position, padding masked, and tokens of type 1 (action tokens) visible to each other in both directions
  (modeling_qwen2_5_vl_act.py:560-732).
* ``prepare_inputs_for_generation``: what one decoding step feeds the model -- ids and token types sliced to the
  new positions, pixels only on the first step (modeling_qwen2_5_vl_act.py:2019-2171).
* ``_get_image_nums_and_video_nums`` / ``_expand_inputs_for_generation``: per-sample vision item counts and the
  ``num_return_sequences`` expansion of ids and per-sample slices of the packed vision tensors
  (modeling_qwen2_5_vl_act.py:2173-2336).
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch


# ----------------------------------------------------------------------------- dense mask rule
def causal_mask_with_cache_position(attention_mask: Optional[torch.Tensor], sequence_length: int, target_length: int,
                                    dtype: torch.dtype, device, cache_position: torch.Tensor, batch_size: int,
                                    config=None, past_key_values=None) -> torch.Tensor:
    """Additive mask ``[B, 1, sequence_length, target_length]``: key j is visible to the query at cache position p
    when ``j <= p`` and key j is not padding. A 4-D ``attention_mask`` is returned unchanged."""
    if attention_mask is not None and attention_mask.dim() == 4:
        return attention_mask
    lowest = torch.finfo(dtype).min
    keys = torch.arange(target_length, device=device)
    hidden = keys.view(1, -1) > cache_position.to(device).view(-1, 1)  # [Q, K]
    window = getattr(config, "sliding_window", None) if config is not None and getattr(config, "use_sliding_window", False) else None
    if window:
        hidden = hidden | (keys.view(1, -1) <= cache_position.to(device).view(-1, 1) - int(window))
    mask = torch.zeros((sequence_length, target_length), dtype=dtype, device=device).masked_fill(hidden, lowest)
    mask = mask[None, None].expand(batch_size, 1, -1, -1).clone()
    if attention_mask is not None:
        n = min(attention_mask.shape[-1], target_length)
        pad = (attention_mask[:, :n].to(device) == 0)[:, None, None, :]
        mask[..., :n] = mask[..., :n].masked_fill(pad, lowest)
    return mask


def dense_attention_mask(attention_mask: Optional[torch.Tensor], input_tensor: torch.Tensor, cache_position: torch.Tensor,
                         past_seen: int = 0, moe_token_types: Optional[torch.Tensor] = None, config=None) -> torch.Tensor:
    """The full rule for a ``[B, Q, C]`` input whose queries sit at ``cache_position``: causal + padding, then every
    pair of type-1 tokens is opened in both directions."""
    B, Q = input_tensor.shape[0], input_tensor.shape[1]
    target = max(past_seen + Q, int(attention_mask.shape[-1]) if attention_mask is not None else 0)
    mask = causal_mask_with_cache_position(attention_mask, Q, target, input_tensor.dtype, input_tensor.device, cache_position, B,
                                           config=config)
    if moe_token_types is not None:
        t1 = (moe_token_types.to(input_tensor.device) == 1)
        keys = t1[:, None, None, :target]  # [B, 1, 1, K]
        if keys.shape[-1] < target:
            keys = torch.nn.functional.pad(keys, (0, target - keys.shape[-1]))
        queries = t1.index_select(1, cache_position.to(t1.device).clamp(max=t1.shape[1] - 1))[:, None, :, None]  # [B, 1, Q, 1]
        mask = torch.where(queries & keys, torch.zeros_like(mask), mask)
    return mask


class MoEModelMaskMixin:
    """Method names of the reference's decoder stack for the dense mask."""

    def _update_causal_mask(self, attention_mask, input_tensor, cache_position, past_key_values=None, output_attentions=False,
                            moe_token_types=None):
        past = 0
        if past_key_values is not None and hasattr(past_key_values, "get_seq_length"):
            past = int(past_key_values.get_seq_length())
        return dense_attention_mask(attention_mask, input_tensor, cache_position, past, moe_token_types, getattr(self, "config", None))

    @staticmethod
    def _prepare_4d_causal_attention_mask_with_cache_position(attention_mask, sequence_length, target_length, dtype, device,
                                                              cache_position, batch_size, config=None, past_key_values=None):
        return causal_mask_with_cache_position(attention_mask, sequence_length, target_length, dtype, device, cache_position,
                                               batch_size, config, past_key_values)


# ----------------------------------------------------------------------------- generation hooks
class GenerationHooksMixin:
    """Method names of the reference's top model for Hugging Face style generation loops."""

    def prepare_inputs_for_generation(self, input_ids, past_key_values=None, attention_mask=None, inputs_embeds=None,
                                      moe_token_types=None, cache_position=None, position_ids=None, use_cache=True,
                                      pixel_values=None, pixel_values_videos=None, image_grid_thw=None, video_grid_thw=None,
                                      second_per_grid_ts=None, dataset_names=None, proprioception=None, dof_mask=None,
                                      agent_pos_mask=None, **kwargs) -> Dict[str, Any]:
        if moe_token_types is None:  # plain text / VQA generation: every token goes to the VLM expert
            moe_token_types = torch.zeros_like(input_ids)
        if cache_position is None:
            past = int(past_key_values.get_seq_length()) if past_key_values is not None and hasattr(past_key_values, "get_seq_length") else 0
            cache_position = torch.arange(past, input_ids.shape[1], device=input_ids.device)
        first_step = int(cache_position[0]) == 0
        if past_key_values is not None and not first_step:
            if inputs_embeds is not None:  # embeddings cover the prompt only: later steps use the new ids
                input_ids = input_ids[:, -cache_position.shape[0]:]
            elif input_ids.shape[1] != cache_position.shape[0]:
                input_ids = input_ids.index_select(1, cache_position)
            if moe_token_types.shape[1] != cache_position.shape[0]:
                if moe_token_types.shape[1] > int(cache_position[-1]):
                    moe_token_types = moe_token_types.index_select(1, cache_position)
                else:  # generated tokens are text
                    moe_token_types = moe_token_types.new_zeros((moe_token_types.shape[0], cache_position.shape[0]))
        if not first_step:  # the vision tower and the proprioception embedding run once, with the prompt
            pixel_values = pixel_values_videos = None
        inputs: Dict[str, Any] = {"inputs_embeds": inputs_embeds, "input_ids": None} if (inputs_embeds is not None and first_step) \
            else {"input_ids": input_ids, "inputs_embeds": None}
        inputs.update({"position_ids": None if first_step else position_ids, "past_key_values": past_key_values, "use_cache": use_cache,
                       "attention_mask": attention_mask, "moe_token_types": moe_token_types, "cache_position": cache_position,
                       "pixel_values": pixel_values, "pixel_values_videos": pixel_values_videos, "image_grid_thw": image_grid_thw,
                       "video_grid_thw": video_grid_thw, "second_per_grid_ts": second_per_grid_ts, "dataset_names": dataset_names,
                       "proprioception": proprioception, "dof_mask": dof_mask, "agent_pos_mask": agent_pos_mask})
        return inputs

    def _get_image_nums_and_video_nums(self, input_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Images and videos per sample: a vision-start token followed by an image / video placeholder."""
        cfg = self.config
        after_start = torch.zeros_like(input_ids, dtype=torch.bool)
        after_start[:, 1:] = input_ids[:, :-1] == cfg.vision_start_token_id
        return ((input_ids == cfg.image_token_id) & after_start).sum(1), ((input_ids == cfg.video_token_id) & after_start).sum(1)

    def _expand_inputs_for_generation(self, expand_size: int = 1, is_encoder_decoder: bool = False,
                                      input_ids: Optional[torch.Tensor] = None, **model_kwargs):
        """Repeat every sample ``expand_size`` times: ids and per-sample tensors by ``repeat_interleave``; the packed
        vision tensors (all samples' patches / grids concatenated) sample by sample."""
        if expand_size == 1:
            return input_ids, model_kwargs
        img_n, vid_n = self._get_image_nums_and_video_nums(input_ids)

        def repeat_packed(values: torch.Tensor, lengths) -> torch.Tensor:
            parts = torch.split(values, [int(n) for n in lengths])
            return torch.cat([p for p in parts for _ in range(expand_size)], dim=0)

        out = dict(model_kwargs)
        for grid_key, pix_key, counts in (("image_grid_thw", "pixel_values", img_n), ("video_grid_thw", "pixel_values_videos", vid_n)):
            grid = model_kwargs.get(grid_key)
            if grid is None:
                continue
            per_item = grid.prod(dim=1)  # patches of every image / video
            per_sample = [int(s.sum()) for s in torch.split(per_item, [int(n) for n in counts])]
            if model_kwargs.get(pix_key) is not None:
                out[pix_key] = repeat_packed(model_kwargs[pix_key], per_sample)
            out[grid_key] = repeat_packed(grid, counts)
        if model_kwargs.get("second_per_grid_ts") is not None:
            ts = model_kwargs["second_per_grid_ts"]
            ts = ts if isinstance(ts, torch.Tensor) else torch.as_tensor(ts)
            out["second_per_grid_ts"] = repeat_packed(ts, vid_n)
        B = input_ids.shape[0]
        for k, v in model_kwargs.items():
            if k in ("image_grid_thw", "pixel_values", "video_grid_thw", "pixel_values_videos", "second_per_grid_ts", "cache_position"):
                continue
            if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.shape[0] == B:
                out[k] = v.repeat_interleave(expand_size, dim=0)
            elif isinstance(v, list) and len(v) == B:
                out[k] = [x for x in v for _ in range(expand_size)]
        return input_ids.repeat_interleave(expand_size, dim=0), out

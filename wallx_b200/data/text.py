"""Prompt construction, image-placeholder expansion, tokenisation and label masking.

Restates the behaviour of the reference's ``wall_x/data/utils.py``: prompt template
(:414-503), per-frame instruction lookup (:320-363), priority sampling of instruction parts
(:366-411), ``<point>`` rescaling (:240-317), FAST token substitution (:506-611) and
``preprocesser_call`` (:70-237: ``<|image_pad|>`` expansion to ``prod(thw)/merge^2`` tokens,
assistant-only labels with ``<|action|>``, ``<|propri|>`` and padding masked out, ``labels=None``
when nothing is left to learn).

Label regions are found on token ids (between ``<|im_start|> assistant \\n`` and the next
``<|im_end|>`` inclusive, plus the token after it) instead of re-tokenising text fragments, which
gives the same spans and is independent of the tokenizer's merges.
"""
from __future__ import annotations

import random
import re
from collections import OrderedDict
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .config import MULTIMODAL_DATASET_NAMES

CAMERA_NAME_MAPPING = {
    "face_view": "front view", "left_wrist_view": "left wrist view", "right_wrist_view": "right wrist view",
    "move1_view": "move view", "move2_view": "move view", "wall_view": "wall view", "top_view": "top view",
}

# control frequency -> number of action steps tokenised by FAST, per dataset
FREQUENCY_MAPPING = {
    "x2_normal": 32, "fractal": 5, "bridge_data_v2": 5, "droid": 15, "agibotworld_alpha": 32, "DobbE": 30, "RH20T": 10,
    "UMI-biarm": 10, "austin_buds": 20, "austin_sailor": 20, "austin_sirius": 20, "bc_z": 10,
    "berkeley_autolab_ur5": 5, "berkeley_cable_routing": 10, "berkeley_fanuc_manipulation": 10,
    "dlr_edan_shared_control": 5, "fmb": 10, "furniture_bench": 10, "jaco_play": 10, "nyu_rot": 10,
    "stanford_hydra": 10, "stanford_kuka_multimodal": 20, "taco_play": 30, "utaustin_mutex": 20, "viola": 20,
}

IM_START, IM_END = "<|im_start|>", "<|im_end|>"
VISION_START, VISION_END, IMAGE_PAD, VIDEO_PAD = "<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>"
PROPRI, ACTION, ACTION_FAST = "<|propri|>", "<|action|>", "<|action_fast|>"
_SUBTASK_KEYS = ("subtask_generation", "distribute")


# ------------------------------------------------------------------------------ instructions
def get_frame_instruction(instruction_info: Dict[str, Any], frame_idx: Optional[int] = None,
                          truncate_keys: Optional[Sequence[str]] = None) -> Tuple[Dict[str, Any], Optional[int]]:
    """Resolve ``{"a b": text}`` frame-range dictionaries to the entry that covers ``frame_idx``."""
    if truncate_keys is None:
        truncate_keys = ("subtask_generation", "distribute", "subtask_generation_zh", "distribute_zh")
    resolved: Dict[str, Any] = {}
    split_end = None
    for key, value in instruction_info.items():
        if not isinstance(value, dict):
            resolved[key] = value
            continue
        for span, text in value.items():
            lo, hi = (int(v) for v in span.split(" "))
            if lo <= frame_idx < hi or lo == frame_idx:
                resolved[key] = text
                if split_end is None and key in truncate_keys:
                    split_end = hi + 1
                break
    return resolved, split_end


def get_task_instruction(frame_instruction_info: Dict[str, Any], priority_order: Optional[Dict[str, float]] = None,
                         rng: Optional[random.Random] = None) -> str:
    """First available priority field always; further ones with their probability; else ``instruction``."""
    rng = rng or random
    order = OrderedDict(priority_order) if priority_order is not None else OrderedDict(
        (k, 0.25) for k in ("subtask_generation", "subtask_generation_zh", "distribute", "distribute_zh"))
    text, got = "", False
    for key, prob in order.items():
        if frame_instruction_info.get(key, "") == "":
            continue
        if got and rng.random() >= prob:
            continue
        text += f"\n{frame_instruction_info[key]}"
        got = True
        break
    return text if got else frame_instruction_info.get("instruction", "")


def get_wallx_normal_text(instruction_info: Dict[str, Any], action_chunk_size: int, frame_idx: int,
                          priority_order: Optional[Dict[str, float]] = None, cam_mapping: Optional[Dict[str, str]] = None,
                          generate_subtask_ratio: float = 0.0, rng: Optional[random.Random] = None) -> Tuple[str, bool]:
    """The Wall-X chat prompt: system prologue, observation with one image slot per camera,
    instruction, proprioception slot, and the assistant turn (FAST slot + ``<|action|>`` x chunk)."""
    rng = rng or random
    head = f"{IM_START}system\nYou are a helpful assistant.{IM_END}\n"
    user = f"{IM_START}user\nObservation:"
    for cam in (cam_mapping or {}).values():
        user += f" {CAMERA_NAME_MAPPING.get(cam, cam)}: {VISION_START}{IMAGE_PAD}{VISION_END}"
    user += "\nInstruction:"
    frame_info, _ = get_frame_instruction(instruction_info, frame_idx=frame_idx)
    if set(frame_info) & set(_SUBTASK_KEYS) and rng.random() < generate_subtask_ratio:
        instruction = frame_info.get("instruction", "")
        answer = next(frame_info[k] for k in _SUBTASK_KEYS if k in frame_info)
        user += f" {instruction}\nPredict the next action in language.\n{IM_END}\n"
        return head + user + f"{IM_START}assistant\n{answer}\n{IM_END}", True
    instruction = get_task_instruction(frame_info, priority_order, rng)
    user += f" {instruction}\nPredict the next action in robot action.\nProprioception: {PROPRI}\n{IM_END}\n"
    tail = f"{IM_START}assistant\n{ACTION_FAST}{IM_END}\n{ACTION * action_chunk_size}"
    return head + user + tail, False


_POINT = re.compile(r"<point>(.*?)</point>")


def process_grounding_points(text: str, orig_height: int, orig_width: int, resized_height: int, resized_width: int,
                             model_type: str) -> str:
    """Rescale 2- or 4-number ``<point>`` payloads to the resized image (qwen2_5: pixels; qwen2: 0..1000)."""
    if model_type not in ("qwen2", "qwen2_5"):
        raise ValueError(f"Unsupported model type: {model_type}")

    def conv(v: int, orig: int, new: int):
        if model_type == "qwen2_5":
            return max(0, min(round(v * new / orig), new - 1))
        return max(0, min(999.999, v / orig * 1000))

    def repl(m):
        nums = [int(n) for n in re.findall(r"\d+", m.group(1))]
        if len(nums) not in (2, 4):
            return f'<point>[{", ".join(map(str, nums))}]</point>'
        out = [conv(v, orig_width if i % 2 == 0 else orig_height, resized_width if i % 2 == 0 else resized_height)
               for i, v in enumerate(nums)]
        return f'<point>[{", ".join(map(str, out))}]</point>'

    return _POINT.sub(repl, text)


# ------------------------------------------------------------------------------ FAST substitution
def get_action_tokens(normalized_actions, action_tokenizer) -> List[List[str]]:
    out = []
    for a in normalized_actions:
        arr = a.detach().cpu().numpy() if isinstance(a, torch.Tensor) else a
        ids = action_tokenizer(arr)
        out.append([f"<|action_token_{j}|>" for j in ids[0]])
    return out


def pad_action_token_strs(token_lists: List[List[str]], pad_token: str = "<|endoftext|>") -> List[str]:
    width = max(len(t) for t in token_lists)
    return ["".join(t + [f"{IM_END}\n"] + [pad_token] * (width - len(t))) for t in token_lists]


def replace_action_token(text: List[str], norm_action, action_tokenizer, dataset_names: List[str],
                         dof_masks: Optional[torch.Tensor] = None) -> List[str]:
    """FAST mode: the ``<|action_fast|><|im_end|>\\n`` slot becomes the FAST token string and every
    ``<|action|>`` is dropped. Flow mode: the slot is dropped and the ``<|action|>`` run stays."""
    names = [n for n in dataset_names if n not in MULTIMODAL_DATASET_NAMES]
    slot = f"{ACTION_FAST}{IM_END}\n"
    if action_tokenizer is None or norm_action is None:
        return [t.replace(slot, "") for t in text]
    steps = [FREQUENCY_MAPPING.get(n, 32) for n in names]
    chunks = [a[: steps[i], dof_masks[i, 0].bool()] for i, a in enumerate(norm_action)]
    strs = pad_action_token_strs(get_action_tokens(chunks, action_tokenizer))
    out, k = [], 0
    for t in text:
        if ACTION_FAST in t:
            t = t.replace(slot, strs[k])
            k += 1
        out.append(t.replace(ACTION, ""))
    return out


# ------------------------------------------------------------------------------ tokenise + labels
def expand_vision_placeholders(text: List[str], grid_thw, pad_token: str, merge_size: int) -> List[str]:
    if grid_thw is None:
        return text
    unit = merge_size * merge_size
    grids = grid_thw.tolist() if isinstance(grid_thw, torch.Tensor) else list(grid_thw)
    out, k = [], 0
    for t in text:
        parts = t.split(pad_token)
        rebuilt = parts[0]
        for p in parts[1:]:
            if k < len(grids):
                g = grids[k]
                rebuilt += pad_token * (int(g[0]) * int(g[1]) * int(g[2]) // unit)
                k += 1
            else:  # more slots than images: leave the slot as a single token
                rebuilt += pad_token
            rebuilt += p
        out.append(rebuilt)
    return out


def assistant_labels(input_ids: torch.Tensor, tokenizer) -> torch.Tensor:
    """-100 everywhere except assistant turns: from the token after ``<|im_start|>assistant\\n``
    through the closing ``<|im_end|>`` and the token that follows it."""
    labels = torch.full_like(input_ids, -100)
    im_start = tokenizer.convert_tokens_to_ids(IM_START)
    im_end = tokenizer.convert_tokens_to_ids(IM_END)
    marker = tokenizer(f"{IM_START}assistant\n", add_special_tokens=False).input_ids
    m = len(marker)
    for b in range(input_ids.shape[0]):
        row = input_ids[b].tolist()
        i = 0
        while i + m <= len(row):
            if row[i] == im_start and row[i:i + m] == marker:
                start = i + m
                end = None
                for k in range(start, len(row)):
                    if row[k] == im_end:
                        end = min(k + 2, len(row))
                        break
                if end is None:
                    break
                labels[b, start:end] = input_ids[b, start:end]
                i = end
            else:
                i += 1
    return labels


def preprocesser_call(processor, images=None, text=None, videos=None, padding=False, truncation=None,
                      max_length=None, padding_side=None, return_tensors="pt") -> Dict[str, Any]:
    """Images -> patches, placeholder expansion, tokenisation and labels. Returns a plain dict with
    ``input_ids, attention_mask, labels (or None), pixel_values, image_grid_thw`` (+ video twins)."""
    out: Dict[str, Any] = {}
    image_grid = video_grid = None
    if images is not None and len(images) > 0:
        img = processor.image_processor(images=images, videos=None, return_tensors=return_tensors)
        out["pixel_values"], out["image_grid_thw"] = img["pixel_values"], img["image_grid_thw"]
        image_grid = img["image_grid_thw"]
    if videos is not None:
        vid = processor.image_processor(images=None, videos=videos, return_tensors=return_tensors)
        out["pixel_values_videos"], out["video_grid_thw"] = vid["pixel_values_videos"], vid["video_grid_thw"]
        video_grid = vid["video_grid_thw"]
    text = [text] if not isinstance(text, list) else list(text)
    merge = getattr(getattr(processor, "image_processor", None), "merge_size", 2)
    text = expand_vision_placeholders(text, image_grid, IMAGE_PAD, merge)
    text = expand_vision_placeholders(text, video_grid, VIDEO_PAD, merge)
    tok = processor.tokenizer
    enc = tok(text, return_tensors=return_tensors, padding=padding, truncation=truncation, max_length=max_length)
    ids, am = enc["input_ids"], enc["attention_mask"]
    labels = assistant_labels(ids, tok)
    pad_id = tok.pad_token_id if tok.pad_token_id is not None else tok.eos_token_id
    for t in (tok.convert_tokens_to_ids(ACTION), tok.convert_tokens_to_ids(PROPRI), pad_id):
        labels[labels == t] = -100
    labels[am == 0] = -100
    out["input_ids"], out["attention_mask"] = ids, am
    out["labels"] = labels if bool((labels != -100).any()) else None
    return out

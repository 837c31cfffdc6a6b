"""Synthetic tokenizer/processor and batch generators for the named benchmark shapes.

There is no network for datasets or tokenizer files, so benchmarks and tests use: a stand-in
tokenizer that exposes exactly what the model reads from a Wall-X processor
(``convert_tokens_to_ids``, ``init_kwargs['action_token_vocab_size' / 'action_token_start_index']``,
``len``; reference: scripts/merge_tokenizer.py:15-22 and modeling_qwen2_5_vl_act.py:855-878), and
generators that build LeRobot-style batches (keys and shapes of load_lerobot_dataset.py:306-415)
from uniform-random pixels, ids and actions.

Image path: uint8 frames -> resize to a multiple of 28 px -> CLIP mean/std -> frame repeated to the
temporal patch size 2 -> ``[t*h*w, 3*2*14*14]`` patches, the layout of the HF Qwen2-VL image
processor the reference calls (data/utils.py:110-113).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..config import Qwen2_5_VLConfig

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 4 * 28 * 28,
                 max_pixels: int = 16384 * 28 * 28) -> Tuple[int, int]:
    """Round both sides to multiples of ``factor`` keeping the pixel count within bounds."""
    if max(height, width) / min(height, width) > 200:
        raise ValueError("absolute aspect ratio must be smaller than 200")
    h_bar = max(factor, round(height / factor) * factor)
    w_bar = max(factor, round(width / factor) * factor)
    if h_bar * w_bar > max_pixels:
        beta = math.sqrt((height * width) / max_pixels)
        h_bar = math.floor(height / beta / factor) * factor
        w_bar = math.floor(width / beta / factor) * factor
    elif h_bar * w_bar < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h_bar = math.ceil(height * beta / factor) * factor
        w_bar = math.ceil(width * beta / factor) * factor
    return h_bar, w_bar


def images_to_patches(images: torch.Tensor, patch: int = 14, temporal: int = 2, merge: int = 2,
                      out_dtype=torch.float32) -> Tuple[torch.Tensor, List[List[int]]]:
    """uint8 ``[n, H, W, 3]`` -> ``(pixel_values [n*h*w, 3*temporal*patch*patch], grid_thw)``.

    Runs on whatever device ``images`` is on (the benchmark copies uint8 frames to the GPU and
    patchifies there: 12x fewer host-to-device bytes than fp32 patches)."""
    n, H, W, _ = images.shape
    rh, rw = smart_resize(H, W, factor=patch * merge)
    x = images.permute(0, 3, 1, 2).float()
    if (rh, rw) != (H, W):
        x = torch.nn.functional.interpolate(x, size=(rh, rw), mode="bicubic", align_corners=False, antialias=True)
        x = x.clamp_(0, 255)
    mean = torch.tensor(CLIP_MEAN, device=x.device).view(1, 3, 1, 1)
    std = torch.tensor(CLIP_STD, device=x.device).view(1, 3, 1, 1)
    x = (x / 255.0 - mean) / std
    gh, gw = rh // patch, rw // patch
    # [n, C, gh/m, m, p, gw/m, m, p] with the frame repeated along the temporal patch axis
    x = x.view(n, 3, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.permute(0, 2, 5, 3, 6, 1, 4, 7)  # n, gh/m, gw/m, m, m, C, p, p
    x = x.unsqueeze(6).expand(-1, -1, -1, -1, -1, -1, temporal, -1, -1)  # ..., C, T, p, p
    x = x.reshape(n * gh * gw, 3 * temporal * patch * patch)
    return x.to(out_dtype).contiguous(), [[1, gh, gw] for _ in range(n)]


class SyntheticTokenizer:
    """Minimal tokenizer: named special tokens + an id range for FAST action tokens."""

    def __init__(self, base_vocab: int, action_vocab: int, image_token_id: int, video_token_id: int,
                 vision_start_token_id: int, vision_end_token_id: int, pad_token_id: int = 0, eos_token_id: int = 1,
                 im_start_id: int = 2, assistant_id: int = 3, im_end_id: int = 4):
        self.base_vocab = base_vocab
        self.special = {
            "<|image_pad|>": image_token_id, "<|video_pad|>": video_token_id, "<|vision_start|>": vision_start_token_id,
            "<|vision_end|>": vision_end_token_id, "<|propri|>": base_vocab, "<|action|>": base_vocab + 1,
            "<|im_start|>": im_start_id, "assistant": assistant_id, "<|im_end|>": im_end_id,
        }
        self.action_start = base_vocab + 2
        self.init_kwargs = {"action_token_vocab_size": action_vocab, "action_token_start_index": self.action_start}
        self.pad_token_id = pad_token_id
        self.eos_token_id = eos_token_id
        self.padding_side = "left"
        self._len = base_vocab + 2 + action_vocab

    def __len__(self):
        return self._len

    def add_tokens(self, new_tokens) -> int:
        """Append named tokens after the current vocabulary (consecutive ids); returns how many were new."""
        added = 0
        count = self._len - self.action_start if self._len > self.action_start else 0  # FAST ids already present
        for t in new_tokens:
            if t in self.special:
                continue
            if t.startswith("<|action_token_") and t.endswith("|>"):
                if int(t[len("<|action_token_"):-2]) < count:
                    continue
                if count == 0:
                    self.action_start = self._len
                count += 1
            else:
                if count:
                    raise ValueError("named tokens must be added before the FAST id range")
                self.special[t] = self._len
            self._len += 1
            added += 1
        return added

    def convert_tokens_to_ids(self, token):
        if isinstance(token, (list, tuple)):
            return [self.convert_tokens_to_ids(t) for t in token]
        if token in self.special:
            return self.special[token]
        if token.startswith("<|action_token_") and token.endswith("|>"):
            return self.action_start + int(token[len("<|action_token_"):-2])
        raise KeyError(token)

    # ---- string tokenisation (special tokens are atoms; other text is hashed word by word)
    _SPLIT = None

    def _encode(self, text: str):
        import re
        import zlib

        if SyntheticTokenizer._SPLIT is None:
            SyntheticTokenizer._SPLIT = re.compile(r"(<\|[^|<>]*\|>)")
        ids = []
        for piece in SyntheticTokenizer._SPLIT.split(text):
            if not piece:
                continue
            if piece.startswith("<|") and piece.endswith("|>"):
                if piece in self.special:
                    ids.append(self.special[piece])
                    continue
                if piece.startswith("<|action_token_"):
                    ids.append(self.action_start + int(piece[len("<|action_token_"):-2]))
                    continue
                if piece == "<|endoftext|>":
                    ids.append(self.pad_token_id)
                    continue
            for word in re.findall(r"\n|[A-Za-z0-9_]+|[^\sA-Za-z0-9_]", piece):
                if word == "assistant":
                    ids.append(self.special["assistant"])
                elif word == "\n":
                    ids.append(5)
                else:
                    ids.append(6 + zlib.crc32(word.encode()) % max(1, self.text_hi - 6))
        return ids

    @property
    def text_hi(self):
        lows = [v for v in self.special.values() if v > 6]
        return min(min(lows), self.base_vocab) if lows else self.base_vocab

    def encode(self, text, add_special_tokens=False):
        return self._encode(text)

    def __call__(self, text, return_tensors=None, padding=False, truncation=None, max_length=None,
                 add_special_tokens=False):
        single = isinstance(text, str)
        rows = [self._encode(t) for t in ([text] if single else text)]
        if truncation and max_length:
            rows = [r[:max_length] for r in rows]
        if single and return_tensors is None:
            return type("Enc", (), {"input_ids": rows[0]})()
        width = max(len(r) for r in rows)
        ids = torch.full((len(rows), width), self.pad_token_id, dtype=torch.long)
        am = torch.zeros((len(rows), width), dtype=torch.long)
        for i, r in enumerate(rows):
            if self.padding_side == "left":
                ids[i, width - len(r):] = torch.tensor(r, dtype=torch.long)
                am[i, width - len(r):] = 1
            else:
                ids[i, : len(r)] = torch.tensor(r, dtype=torch.long)
                am[i, : len(r)] = 1
        return {"input_ids": ids, "attention_mask": am}

    def decode(self, ids, **kw):
        inv = {v: k for k, v in self.special.items()}
        out = []
        for i in (ids.tolist() if isinstance(ids, torch.Tensor) else ids):
            if i in inv:
                out.append(inv[i])
            elif i >= self.action_start:
                out.append(f"<|action_token_{i - self.action_start}|>")
            else:
                out.append(f"<{i}>")
        return "".join(out)

    def batch_decode(self, batch, **kw):
        return [self.decode(row) for row in batch]


class SyntheticImageProcessor:
    """uint8 HWC arrays / PIL images -> Qwen2-VL style patches (see :func:`images_to_patches`)."""

    def __init__(self, patch_size=14, temporal_patch_size=2, merge_size=2):
        self.patch_size, self.temporal_patch_size, self.merge_size = patch_size, temporal_patch_size, merge_size

    def __call__(self, images=None, videos=None, return_tensors="pt"):
        import numpy as np

        pvs, grids = [], []
        for im in images or []:
            arr = im if torch.is_tensor(im) else torch.as_tensor(np.array(im))
            if arr.dim() == 3 and arr.shape[0] == 3 and arr.shape[-1] != 3:
                arr = arr.permute(1, 2, 0)
            if arr.dtype != torch.uint8:
                arr = (arr.float().clamp(0, 1) * 255).to(torch.uint8) if arr.is_floating_point() else arr.to(torch.uint8)
            pv, g = images_to_patches(arr.unsqueeze(0), self.patch_size, self.temporal_patch_size, self.merge_size)
            pvs.append(pv)
            grids.extend(g)
        return {"pixel_values": torch.cat(pvs) if pvs else None,
                "image_grid_thw": torch.tensor(grids, dtype=torch.long) if grids else None}


class SyntheticProcessor:
    def __init__(self, tokenizer: SyntheticTokenizer, image_processor=None):
        self.tokenizer = tokenizer
        self.image_processor = image_processor or SyntheticImageProcessor()
        self.action_processor = None

    def batch_decode(self, batch, **kw):
        return self.tokenizer.batch_decode(batch, **kw)

    def apply_chat_template(self, messages, tokenize: bool = False, add_generation_prompt: bool = True) -> str:
        """Qwen chat layout: ``<|im_start|>role\n ... <|im_end|>\n`` with one vision span per image item."""
        out = []
        for m in messages:
            out.append(f"<|im_start|>{m['role']}\n")
            content = m["content"]
            if isinstance(content, str):
                out.append(content)
            else:
                for item in content:
                    if item.get("type") == "image":
                        out.append("<|vision_start|><|image_pad|><|vision_end|>")
                    elif item.get("type") == "text":
                        out.append(item["text"])
            out.append("<|im_end|>\n")
        if add_generation_prompt:
            out.append("<|im_start|>assistant\n")
        text = "".join(out)
        return self.tokenizer.encode(text) if tokenize else text

    def __call__(self, text=None, images=None, return_tensors="pt", padding=True, **kw):
        """Image patches + tokenised text with every ``<|image_pad|>`` expanded to its image's token count."""
        texts = [text] if isinstance(text, str) else list(text)
        out = {}
        if images:
            img = self.image_processor(images=images, return_tensors=return_tensors)
            out.update(img)
            merge2 = self.image_processor.merge_size ** 2
            counts = [int(g.prod()) // merge2 for g in img["image_grid_thw"]]
            k = 0
            expanded = []
            for t in texts:
                while "<|image_pad|>" in t and k < len(counts):
                    t = t.replace("<|image_pad|>", "<|placeholder|>" * counts[k], 1)
                    k += 1
                expanded.append(t.replace("<|placeholder|>", "<|image_pad|>"))
            texts = expanded
        out.update(self.tokenizer(texts, return_tensors=return_tensors, padding=padding))
        return out

    def save_pretrained(self, directory: str) -> None:
        import json
        import os

        os.makedirs(directory, exist_ok=True)
        tok = self.tokenizer
        with open(os.path.join(directory, "synthetic_tokenizer.json"), "w") as f:
            json.dump({"base_vocab": tok.base_vocab, "special": tok.special, "init_kwargs": tok.init_kwargs,
                       "length": len(tok), "padding_side": tok.padding_side}, f, indent=1)


def make_processor(config: Qwen2_5_VLConfig, action_vocab: int) -> SyntheticProcessor:
    """Tokenizer whose length equals ``config.vocab_size`` (base + <|propri|> + <|action|> + FAST ids)."""
    base = config.vocab_size - 2 - action_vocab
    tok = SyntheticTokenizer(base, action_vocab, config.image_token_id, config.video_token_id,
                             config.vision_start_token_id, config.vision_end_token_id,
                             pad_token_id=config.pad_token_id if config.pad_token_id is not None else 0)
    proc = SyntheticProcessor(tok)
    if action_vocab >= 3:
        from .fast_tokenizer import DctActionTokenizer

        proc.action_processor = DctActionTokenizer(action_vocab)
    return proc


def _text_ids(n: int, hi: int, forbidden: Sequence[int], gen: torch.Generator) -> torch.Tensor:
    ids = torch.randint(5, hi, (n,), generator=gen)
    for f in forbidden:
        ids = torch.where(ids == f, torch.full_like(ids, 5), ids)
    return ids


def make_batch(config: Qwen2_5_VLConfig, processor: SyntheticProcessor, batch: int, views: int = 3,
               image_hw: Tuple[int, int] = (256, 256), prompt_len: int = 64, horizon: int = 32, mode: str = "flow",
               fast_tokens: int = 48, generator: Optional[torch.Generator] = None, raw_images: bool = False,
               pad_to: Optional[int] = None, dataset_name: str = "x2_normal") -> Dict[str, object]:
    """One synthetic LeRobot-style batch on the CPU.

    ``mode="flow"``: ``horizon`` ``<|action|>`` tokens end each sample, no labels (flow MSE only).
    ``mode="fast"``: ``fast_tokens`` FAST ids form the assistant turn with next-token labels on them.
    ``raw_images=True`` keeps ``images_uint8 [B*views, H, W, 3]`` instead of ``pixel_values`` so that
    patchifying can happen after the host-to-device copy.
    """
    gen = generator or torch.Generator().manual_seed(0)
    tok = processor.tokenizer
    A = sum(config.dof_config.values())
    P = sum(config.agent_pos_config.values())
    vc = config.vision_config
    merge = vc.spatial_merge_size
    rh, rw = smart_resize(image_hw[0], image_hw[1], factor=vc.patch_size * merge)
    n_img_tok = (rh // vc.patch_size // merge) * (rw // vc.patch_size // merge)
    special = [config.image_token_id, config.video_token_id, config.vision_start_token_id, config.vision_end_token_id]
    text_hi = min(tok.base_vocab, min(special)) if min(special) > 5 else tok.base_vocab
    rows, labels_rows, type_rows = [], [], []
    for _ in range(batch):
        parts = []
        per_view = max(1, prompt_len // (views + 1))
        for _v in range(views):
            parts.append(_text_ids(per_view, text_hi, special, gen))
            parts.append(torch.tensor([config.vision_start_token_id] + [config.image_token_id] * n_img_tok +
                                      [config.vision_end_token_id]))
        parts.append(_text_ids(prompt_len - per_view * views, text_hi, special, gen))
        parts.append(torch.tensor([tok.convert_tokens_to_ids("<|propri|>")]))
        prompt = torch.cat(parts)
        if mode == "flow":
            tail = torch.full((horizon,), tok.convert_tokens_to_ids("<|action|>"))
            ids = torch.cat([prompt, tail])
            lab = None
            types = torch.cat([torch.zeros_like(prompt), torch.ones_like(tail)])
        elif mode == "fast":
            head = torch.tensor([tok.convert_tokens_to_ids("<|im_start|>"), tok.convert_tokens_to_ids("assistant")])
            fast = torch.randint(0, tok.init_kwargs["action_token_vocab_size"], (fast_tokens,), generator=gen) + tok.action_start
            end = torch.tensor([tok.convert_tokens_to_ids("<|im_end|>")])
            ids = torch.cat([prompt, head, fast, end])
            lab = torch.cat([torch.full_like(prompt, -100), torch.full_like(head, -100), fast, end])
            types = torch.zeros_like(ids)
        else:
            raise ValueError(mode)
        rows.append(ids)
        labels_rows.append(lab)
        type_rows.append(types)
    S = max(r.numel() for r in rows)
    if pad_to is not None:
        S = max(S, pad_to)
    pad_id = tok.pad_token_id
    input_ids = torch.full((batch, S), pad_id, dtype=torch.long)
    attn = torch.zeros((batch, S), dtype=torch.long)
    moe = torch.zeros((batch, S), dtype=torch.long)
    labels = torch.full((batch, S), -100, dtype=torch.long) if mode == "fast" else None
    for b, r in enumerate(rows):  # left padding, as the reference's collator (padding_side default "left")
        n = r.numel()
        input_ids[b, S - n:] = r
        attn[b, S - n:] = 1
        moe[b, S - n:] = type_rows[b]
        if labels is not None:
            labels[b, S - n:] = labels_rows[b]
    images = torch.randint(0, 256, (batch * views, image_hw[0], image_hw[1], 3), generator=gen, dtype=torch.uint8)
    out: Dict[str, object] = {
        "input_ids": input_ids, "attention_mask": attn, "moe_token_types": moe,
        "proprioception": torch.randn((batch, 1, P), generator=gen),
        "agent_pos_mask": torch.ones((batch, 1, P)),
        "dataset_names": [dataset_name] * batch,
        "frame_index": torch.zeros(batch, dtype=torch.long),
    }
    if labels is not None:
        out["labels"] = labels
    if mode == "flow":
        out["action_chunk"] = torch.rand((batch, horizon, A), generator=gen) * 2 - 1
        out["dof_mask"] = torch.ones((batch, horizon, A))
    if raw_images:
        out["images_uint8"] = images
        gh, gw = rh // vc.patch_size, rw // vc.patch_size
        out["image_grid_thw"] = torch.tensor([[1, gh, gw]] * (batch * views), dtype=torch.long)
    else:
        pv, grid = images_to_patches(images, vc.patch_size, vc.temporal_patch_size, merge)
        out["pixel_values"] = pv
        out["image_grid_thw"] = torch.tensor(grid, dtype=torch.long)
    return out

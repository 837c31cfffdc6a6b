"""Checkpoint I/O: HF-compatible safetensors (single or sharded + index) and training state.

* Pretrained / exported weights use the reference's key layout (modeling_qwen2_5_vl_act.py:785-794
  reads every ``*.safetensors`` of a directory), so ``from_pretrained`` round-trips with Wall-X
  checkpoints.
* Training checkpoints are one file per rank (fp32 master shard, Adam moments, step, RNG, sampler
  position, LR-schedule state) plus a manifest that records the world size and flat-parameter
  layout, so that a run can resume on a different number of GPUs (``parallel/reshard.py``).
"""
from __future__ import annotations

import glob
import json
import os
from typing import Dict, Iterable, List

import torch


def load_safetensors_dir(directory: str, device: str = "cpu") -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    files = sorted(glob.glob(os.path.join(directory, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no *.safetensors under {directory}")
    state: Dict[str, torch.Tensor] = {}
    for f in files:
        state.update(load_file(f, device=device))
    return state


def save_safetensors_sharded(state: Dict[str, torch.Tensor], directory: str, max_shard_bytes: int = 4 << 30) -> List[str]:
    """Write ``model.safetensors`` or ``model-0000i-of-0000n.safetensors`` + ``model.safetensors.index.json``."""
    from safetensors.torch import save_file

    os.makedirs(directory, exist_ok=True)
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    for k, v in state.items():
        t = v.detach().to("cpu").contiguous()
        nbytes = t.numel() * t.element_size()
        if size + nbytes > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][k] = t
        size += nbytes
    names = []
    if len(shards) == 1:
        names = ["model.safetensors"]
        save_file(shards[0], os.path.join(directory, names[0]), metadata={"format": "pt"})
        return names
    index = {"metadata": {"total_size": 0}, "weight_map": {}}
    for i, sh in enumerate(shards):
        name = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        names.append(name)
        save_file(sh, os.path.join(directory, name), metadata={"format": "pt"})
        for k, t in sh.items():
            index["weight_map"][k] = name
            index["metadata"]["total_size"] += t.numel() * t.element_size()
    with open(os.path.join(directory, "model.safetensors.index.json"), "w", encoding="utf-8") as f:
        json.dump(index, f, indent=1)
    return names


def rename_qwen_to_moe(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Stock Qwen2.5-VL keys -> this model: ``layers.N.mlp.`` becomes ``layers.N.moe.experts.0.``
    (reference: qwen_vl_act_trainer.py:633-697)."""
    out = {}
    for k, v in state.items():
        if ".layers." in k and ".mlp." in k and k.startswith("model."):
            k = k.replace(".mlp.", ".moe.experts.0.")
        out[k] = v
    return out


def strip_prefixes(state: Dict[str, torch.Tensor], prefixes: Iterable[str] = ("module.", "_orig_mod.")) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in state.items():
        changed = True
        while changed:
            changed = False
            for p in prefixes:
                if k.startswith(p):
                    k = k[len(p):]
                    changed = True
        out[k] = v
    return out

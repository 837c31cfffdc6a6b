"""Resharding of optimizer state between world sizes.

A training checkpoint holds one ``optim_rank<r>_of_<w>.pt`` per rank with that rank's shard of
every flat buffer (fp32 master, Adam moments). To resume on another number of ranks the shards of
each buffer are concatenated in rank order, cut to the buffer's true length and re-sliced for the
new layout. (The reference can only resume model weights on its FSDP2 path,
qwen_vl_act_trainer.py:797-837; optimizer, scheduler and step are not restored there.)
"""
from __future__ import annotations

import os

import torch


def _shard_file(path: str, rank: int, world: int) -> str:
    return os.path.join(path, f"optim_rank{rank:05d}_of_{world:05d}.pt")


def load_optimizer_shards(engine, path: str, old_world: int) -> None:
    files = [_shard_file(path, r, old_world) for r in range(old_world)]
    for f in files:
        if not os.path.exists(f):
            raise FileNotFoundError(f"checkpoint shard missing: {f}")
    states = [torch.load(f, map_location="cpu", weights_only=False) for f in files]
    layouts = states[0]["layout"]
    if len(layouts) != len(engine.buffers):
        raise ValueError("checkpoint has a different number of flat buffers than the model")
    engine.optimizer.step_count = int(states[0]["opt"]["step"])
    for i, b in enumerate(engine.buffers):
        name, numel, padded_old, _ = layouts[i]
        if numel != b.numel:
            raise ValueError(f"buffer {name}: {numel} elements in the checkpoint, {b.numel} in the model")
        for key, dst in (("master", b.master), ("exp_avg", b.exp_avg), ("exp_avg_sq", b.exp_avg_sq)):
            full = torch.cat([s["opt"]["buffers"][i][key].reshape(-1).float() for s in states])[:numel]
            if b.padded > numel:
                full = torch.cat([full, full.new_zeros(b.padded - numel)])
            s0, s1 = b.shard_range
            dst.copy_(full[s0:s1].to(dst.dtype))
    if "rng" in states[min(engine.rank, old_world - 1)]:
        rng = states[min(engine.rank, old_world - 1)]["rng"]
        try:
            torch.set_rng_state(rng["torch"])
        except Exception:
            pass

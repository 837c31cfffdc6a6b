"""Resharding of optimizer state between world sizes.

A training checkpoint holds one ``optim_rank<r>_of_<w>.pt`` per rank with that rank's shard of
every buffer (fp32 master, Adam moments) and the layout that says where each parameter sits in it
(a contiguous range of a flat buffer, or the same rows of every weight of a row-sharded unit). To
resume, the whole state of every parameter is rebuilt by name and re-cut for the new layout: another
world size, or the other parameter plan. (The reference can only resume model weights on its FSDP2 path,
qwen_vl_act_trainer.py:797-837; optimizer, scheduler and step are not restored there.)
"""
from __future__ import annotations

import os

import torch


def _shard_file(path: str, rank: int, world: int) -> str:
    return os.path.join(path, f"optim_rank{rank:05d}_of_{world:05d}.pt")


def _param_spans(entry):
    """``[(name, offset, numel, shape or None)]`` of one layout entry (old entries carry no shapes)."""
    name, numel, _padded, items = entry[0], entry[1], entry[2], entry[3]
    shapes = entry[5] if len(entry) > 5 else None
    kind = entry[4] if len(entry) > 4 else "flat"
    out = []
    for k, (pname, off) in enumerate(items):
        if shapes is not None:
            shape = tuple(shapes[k])
            n = 1
            for d in shape:
                n *= int(d)
        else:
            nxt = min([o for _, o in items if o > off] + [numel])
            shape, n = None, nxt - off
        out.append((pname, int(off), int(n), shape))
    return kind, out


def _full_states(states, key: str, old_world: int):
    """Whole fp32 state vector ``key`` of every parameter, by name, from the per-rank shards of a checkpoint."""
    full = {}
    for i, entry in enumerate(states[0]["layout"]):
        kind, spans = _param_spans(entry)
        shards = [s["opt"]["buffers"][i][key].reshape(-1).float() for s in states]
        if kind == "rows":  # every rank holds rows [r * R / w, (r + 1) * R / w) of each weight at the same shard offset
            for pname, off, n, shape in spans:
                per = n // old_world
                full[pname] = torch.cat([sh[off:off + per] for sh in shards])
        else:
            whole = torch.cat(shards)
            for pname, off, n, shape in spans:
                full[pname] = whole[off:off + n]
    return full


def load_optimizer_shards(engine, path: str, old_world: int) -> None:
    """Fill this rank's optimizer state from a checkpoint written by ``old_world`` ranks. Parameters are matched
    by name, so the checkpoint may come from another world size and from the other parameter plan (resident flat
    buffers or row-sharded units)."""
    files = [_shard_file(path, r, old_world) for r in range(old_world)]
    for f in files:
        if not os.path.exists(f):
            raise FileNotFoundError(f"checkpoint shard missing: {f}")
    states = [torch.load(f, map_location="cpu", weights_only=False) for f in files]
    have = {}
    for entry in states[0]["layout"]:
        for pname, _off, n, _shape in _param_spans(entry)[1]:
            have[pname] = n
    want = {n: p.numel() for b in engine.buffers for n, p in zip(b.names, b.params)}
    if set(have) != set(want):
        diff = sorted(set(have) ^ set(want))
        raise ValueError(f"checkpoint and model disagree on the trained parameters, e.g. {diff[:3]}")
    for n, k in want.items():
        if have[n] != k:
            raise ValueError(f"parameter {n}: {have[n]} elements in the checkpoint, {k} in the model")
    engine.optimizer.step_count = int(states[0]["opt"]["step"])
    for key in ("master", "exp_avg", "exp_avg_sq"):
        full = _full_states(states, key, old_world)
        for b in engine.buffers:
            dst = getattr(b, key)
            dst.zero_()
            if b.kind == "rows":
                for i, (pname, off) in enumerate(zip(b.names, b.offsets)):
                    per = b.shard_len(i)
                    dst[off:off + per].copy_(full[pname][b.rank * per:(b.rank + 1) * per].to(dst.dtype))
            else:
                s0, s1 = b.shard_range
                for pname, p, off in zip(b.names, b.params, b.offsets):
                    lo, hi = max(off, s0), min(off + p.numel(), s1)
                    if hi > lo:
                        dst[lo - s0:hi - s0].copy_(full[pname][lo - off:hi - off].to(dst.dtype))
        del full
    if "rng" in states[min(engine.rank, old_world - 1)]:
        rng = states[min(engine.rank, old_world - 1)]["rng"]
        try:
            torch.set_rng_state(rng["torch"])
        except Exception:
            pass
        if rng.get("cuda") is not None and torch.cuda.is_available():
            try:
                torch.cuda.set_rng_state(rng["cuda"])
            except Exception:
                pass

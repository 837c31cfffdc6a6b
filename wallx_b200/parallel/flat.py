"""Flat parameter / gradient storage and the sharded optimizer state that goes with it.

B200-first memory plan: with 180 GB of HBM per GPU the bf16 parameters (a few GB) stay resident
and whole on every rank; what is sharded across ranks is the expensive part -- fp32 master
weights and both Adam moments (12 bytes per parameter). Each rank owns one contiguous shard of
every flat buffer: gradients are reduce-scattered onto the owner, the owner runs the fused
clip/scale + AdamW kernel on its shard and the new bf16 values are written back into every rank's
resident copy.

Compared with the reference (accelerate FSDP2, bf16 parameters *and* bf16 Adam states,
qwen_vl_act_trainer.py:527,577-581,609-611) this keeps fp32 master weights and moments; set
``master_dtype=torch.bfloat16`` to mimic the reference's numerics.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class ParamSegment:
    """A contiguous run of parameters that share optimizer hyper-parameters."""

    def __init__(self, start: int, end: int, lr_scale: float, weight_decay: float, name: str):
        self.start, self.end, self.lr_scale, self.weight_decay, self.name = start, end, lr_scale, weight_decay, name


class FlatBuffer:
    """One flat bf16 (or fp32 on CPU) buffer holding a list of parameters, its gradient twin and
    this rank's shard of the optimizer state."""

    ALIGN = 1024  # elements; keeps every shard 2 KB aligned for vector and bulk accesses
    kind = "flat"

    def __init__(self, named_params: Sequence[Tuple[str, nn.Parameter]], world: int = 1, rank: int = 0,
                 groups: Optional[Sequence[Tuple[str, float, float]]] = None, name: str = "",
                 alloc=None, master_dtype=torch.float32):
        """``groups``: per parameter ``(group_name, lr_scale, weight_decay)`` in the same order."""
        assert len(named_params) > 0
        self.name = name
        self.world, self.rank = world, rank
        p0 = named_params[0][1]
        self.device, self.dtype = p0.device, p0.dtype
        if groups is None:
            groups = [("default", 1.0, 0.0)] * len(named_params)
        # keep parameters with equal hyper-parameters adjacent
        order = sorted(range(len(named_params)), key=lambda i: (groups[i][0], i))
        self.names: List[str] = []
        self.params: List[nn.Parameter] = []
        self.offsets: List[int] = []
        self.segments: List[ParamSegment] = []
        off = 0
        for i in order:
            n, p = named_params[i]
            g = groups[i]
            if not self.segments or self.segments[-1].name != g[0]:
                self.segments.append(ParamSegment(off, off, g[1], g[2], g[0]))
            self.names.append(n)
            self.params.append(p)
            self.offsets.append(off)
            off += p.numel()
            self.segments[-1].end = off
        self.numel = off
        self.padded = _round_up(off, self.ALIGN * world)
        self.shard_size = self.padded // world
        default = lambda n, dtype: torch.zeros(n, device=self.device, dtype=dtype)
        alloc_param, alloc_grad = alloc if alloc is not None else (default, default)
        self.param = alloc_param(self.padded, self.dtype)
        self.grad = alloc_grad(self.padded, self.dtype)
        with torch.no_grad():
            for p, o in zip(self.params, self.offsets):
                self.param[o:o + p.numel()].copy_(p.data.reshape(-1))
                p.data = self.param[o:o + p.numel()].view(p.shape)
                p.grad = self.grad[o:o + p.numel()].view(p.shape)
        # which parameters received a gradient since the last step (torch's AdamW leaves parameters
        # whose grad is None untouched -- no decay, no moment update -- e.g. the LM head in flow-only
        # training); filled by post-accumulate hooks, merged across ranks by the engine
        self.touched = [False] * len(self.params)
        self._hook_handles = []
        self.on_touch = None  # optional callback(buffer, param_index, kind) used by the engine to overlap the reduction
        for i, p in enumerate(self.params):
            self._hook_handles.append(p.register_post_accumulate_grad_hook(self._make_hook(i, "accumulate")))
        if self.param.is_cuda:  # weight-gradient GEMMs add straight into the flat gradient buffer
            from ..ops import functional as F_

            for i, (p, o) in enumerate(zip(self.params, self.offsets)):
                if p.dim() == 2:
                    F_.register_grad_sink(p, self.grad[o:o + p.numel()].view(p.shape), self._make_hook(i, "sink"))
        self.seg_of_param = []
        for o in self.offsets:
            self.seg_of_param.append(next(k for k, sg in enumerate(self.segments) if sg.start <= o < sg.end))
        s0 = rank * self.shard_size
        self.shard_range = (s0, s0 + self.shard_size)
        self.master = self.param[s0:s0 + self.shard_size].to(master_dtype).clone()
        self.exp_avg = torch.zeros(self.shard_size, device=self.device, dtype=master_dtype)
        self.exp_avg_sq = torch.zeros(self.shard_size, device=self.device, dtype=master_dtype)

    def _make_hook(self, i: int, kind: str = "accumulate"):
        # kind "accumulate": fired by autograd after the gradient kernel was enqueued; kind "sink":
        # fired right after the weight-gradient GEMM that adds into the flat buffer was enqueued
        def hook(_p=None):
            self.touched[i] = True
            cb = self.on_touch
            if cb is not None:
                cb(self, i, kind)

        return hook

    def clear_touched(self) -> None:
        self.touched = [False] * len(self.params)

    def release(self) -> None:
        """Undo the hooks and gradient sinks on the parameters. The hooks are held by the tensors on the C++ side and
        refer back to this buffer, a cycle the garbage collector cannot see: without this call neither the
        parameters nor the optimizer state of a discarded engine are ever freed."""
        for h in self._hook_handles:
            h.remove()
        self._hook_handles = []
        for p in self.params:
            for attr in ("_wx_sink", "_wx_shard"):
                if hasattr(p, attr):
                    delattr(p, attr)
            p.grad = None
        self.on_touch = None

    def update_ranges(self, touched=None) -> List[Tuple[int, int, ParamSegment]]:
        """Shard-local ``(lo, hi, segment)`` ranges to update: touched parameters only, adjacent
        ones with equal hyper-parameters merged."""
        touched = self.touched if touched is None else touched
        if all(touched):
            return self.shard_segments()
        s0, s1 = self.shard_range
        out: List[Tuple[int, int, ParamSegment]] = []
        for i, (p, o) in enumerate(zip(self.params, self.offsets)):
            if not touched[i]:
                continue
            lo, hi = max(o, s0), min(o + p.numel(), s1)
            if hi <= lo:
                continue
            seg = self.segments[self.seg_of_param[i]]
            if out and out[-1][1] == lo - s0 and out[-1][2] is seg:
                out[-1] = (out[-1][0], hi - s0, seg)
            else:
                out.append((lo - s0, hi - s0, seg))
        return out

    def rebind_grads(self) -> None:
        """Point every ``p.grad`` back at the flat gradient buffer (after ``zero_grad(set_to_none)``)."""
        for p, o in zip(self.params, self.offsets):
            p.grad = self.grad[o:o + p.numel()].view(p.shape)

    def zero_grad(self) -> None:
        self.grad.zero_()

    def shard_segments(self) -> List[Tuple[int, int, ParamSegment]]:
        """Intersections of the hyper-parameter segments with this rank's shard, in shard-local
        coordinates (padding elements belong to the last segment; their gradient is zero)."""
        s0, s1 = self.shard_range
        out = []
        for k, seg in enumerate(self.segments):
            a = seg.start
            b = seg.end if k + 1 < len(self.segments) else self.padded
            lo, hi = max(a, s0), min(b, s1)
            if hi > lo:
                out.append((lo - s0, hi - s0, seg))
        return out

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {"master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq}

    # ------------------------------------------------------------------ transport tables
    def rs_segments(self) -> List[Tuple[int, int, int]]:
        """``(offset in the gradient buffer, length, offset in the shard)`` of the pieces this rank reduces."""
        return [(self.shard_range[0], self.shard_size, 0)]

    def push_segments(self) -> List[Tuple[int, int]]:
        """``(offset in the parameter buffer, length)`` of what this rank writes into the peers' copies."""
        return [(self.shard_range[0], self.shard_size)]

"""Sharded data-parallel training engine (the FSDP role of the reference's accelerate setup).

Units follow the reference's ``_no_split_modules`` (one per decoder layer and vision block,
modeling_qwen2_5_vl_act.py:745) plus one root unit; each unit is a :class:`FlatBuffer`.

Per optimizer step: ``accum`` micro-batches of forward/backward accumulate bf16 gradients in the
flat buffers; each unit's gradient is reduce-scattered onto its owner shard (sum in fp32), the
squared global norm is reduced once (one small collective instead of the reference's per-step
clip all-reduce plus ~75 scalar gathers, qwen_vl_act_trainer.py:335-423), then one fused kernel per
shard applies scale + clip + AdamW and the new bf16 values are gathered back into every rank's
resident parameter copy.

Transports: ``"local"`` (one rank), ``"dist"`` (torch.distributed collectives: NCCL on GPUs, gloo
on CPU -- the plain baseline and the CPU test path), ``"symm"`` (hand-written peer-memory kernels
over NVLink, :mod:`wallx_b200.parallel.symm`).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..train.optim import FlatAdamW
from .flat import FlatBuffer


def default_units(model: nn.Module) -> List[Tuple[str, List[Tuple[str, nn.Parameter]]]]:
    """Split trainable parameters into units: vision blocks, decoder layers, root."""
    claimed = set()
    units: List[Tuple[str, List[Tuple[str, nn.Parameter]]]] = []

    def take(prefix: str, mod: nn.Module):
        ps = [(f"{prefix}.{n}", p) for n, p in mod.named_parameters() if p.requires_grad and id(p) not in claimed]
        for _, p in ps:
            claimed.add(id(p))
        if ps:
            units.append((prefix, ps))

    visual = getattr(model, "visual", None)
    if visual is not None:
        for i, blk in enumerate(visual.blocks):
            take(f"visual.blocks.{i}", blk)
    lm = getattr(model, "model", None)
    if lm is not None and hasattr(lm, "layers"):
        for i, layer in enumerate(lm.layers):
            take(f"model.layers.{i}", layer)
    rest = [(n, p) for n, p in model.named_parameters() if p.requires_grad and id(p) not in claimed]
    if rest:
        units.append(("root", rest))
    return units


class TrainEngine:
    def __init__(self, model: nn.Module, lr: float, weight_decay: float = 0.1, betas=(0.9, 0.999), eps: float = 1e-8,
                 max_grad_norm: float = 1.0, grad_accum: int = 1, world: int = 1, rank: int = 0,
                 transport: str = "local", group=None, param_group_fn: Optional[Callable[[str], Tuple[str, float, float]]] = None,
                 master_dtype=torch.float32, symm=None):
        self.model = model
        self.world, self.rank = world, rank
        self.transport = transport if world > 1 else "local"
        self.group = group
        self.symm = symm
        self.grad_accum = grad_accum
        pg = param_group_fn or (lambda name: ("default", 1.0, weight_decay))
        self.buffers: List[FlatBuffer] = []
        units = default_units(model)
        alloc = None
        if self.transport == "symm" and symm is not None:
            align = FlatBuffer.ALIGN * world
            total = sum((sum(p.numel() for _, p in ps) + align - 1) // align * align for _, ps in units)
            symm.reserve(total, dtype=units[0][1][0][1].dtype)
            alloc = (symm.alloc_param, symm.alloc_grad)
        for uname, ps in units:
            groups = [pg(n) for n, _ in ps]
            self.buffers.append(FlatBuffer(ps, world, rank, groups, name=uname, alloc=alloc, master_dtype=master_dtype))
        self.optimizer = FlatAdamW(self.buffers, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                   max_grad_norm=max_grad_norm, grad_accum=grad_accum * world)
        self.last_norm_sq: Optional[torch.Tensor] = None
        # ranks agree on which parameters were used unless batches differ in modality; the merge
        # costs one host read per step, so it can be switched off for homogeneous data
        self.check_touched = True
        if self.transport == "symm":
            symm.register_buffers(self.buffers)
        # Overlap of the gradient reduce-scatter with backward (symmetric transport): a unit is
        # reduced on a side stream as soon as the last of its gradients of the last micro-step has
        # been enqueued. Which parameter comes last, and how many are touched, is learned from the
        # first step; a unit whose pattern differs in a later step is simply reduced after backward.
        self.overlap_reduce = False
        self._micro = 0
        self._armed = False
        self._learned = False
        self._order: Dict[int, list] = {}
        self._trigger: Dict[int, Optional[int]] = {}
        self._expected: Dict[int, int] = {}
        self._seen: Dict[int, set] = {}
        self._early: set = set()
        self._step_begun = False
        self._comm_stream = None
        for k, b in enumerate(self.buffers):
            b.index = k
            b.on_touch = self._on_touch

    # ------------------------------------------------------------------ collectives
    def _reduce_scatter(self) -> Optional[List[torch.Tensor]]:
        if self.transport == "local":
            return None
        if self.transport == "symm":
            if not self.overlap_reduce:
                return self.symm.reduce_scatter_grads(self.buffers)
            if not self._step_begun:  # the last backward did not go through engine.backward(): nothing was overlapped
                self.symm.begin_step()
                self._early = set()
            self._step_begun = False
            # the side stream first: the reductions add to one squared-norm word and must not overlap each other
            if self._comm_stream is not None:
                torch.cuda.current_stream(self.buffers[0].device).wait_stream(self._comm_stream)
            for k in range(len(self.buffers)):  # units that were not reduced during backward
                if k not in self._early:
                    self.symm.reduce_scatter_unit(k)
            if not self._learned and self._order:
                for k, order in self._order.items():
                    self._expected[k] = len({i for i, _ in order})
                    last_i, last_kind = order[-1]
                    self._trigger[k] = last_i if last_kind == "accumulate" else None
                self._learned = True
            return self.symm.grad_shards()
        import torch.distributed as dist

        shards = []
        for b in reversed(self.buffers):
            out = torch.empty(b.shard_size, device=b.device, dtype=b.grad.dtype)
            if b.grad.is_cuda:
                dist.reduce_scatter_tensor(out, b.grad, op=dist.ReduceOp.SUM, group=self.group)
            else:  # gloo has no reduce_scatter: all-reduce and slice
                tmp = b.grad.float()
                dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=self.group)
                out = tmp[b.shard_range[0]:b.shard_range[1]].to(b.grad.dtype)
            shards.append(out)
        return list(reversed(shards))

    def _all_gather_params(self) -> None:
        if self.transport == "local":
            return
        if self.transport == "symm":
            self.symm.all_gather_params(self.buffers)
            return
        import torch.distributed as dist

        for b in self.buffers:
            s0, s1 = b.shard_range
            if b.param.is_cuda:
                dist.all_gather_into_tensor(b.param, b.param[s0:s1].clone(), group=self.group)
            else:
                parts = [torch.empty(b.shard_size, dtype=b.param.dtype) for _ in range(self.world)]
                dist.all_gather(parts, b.param[s0:s1].clone(), group=self.group)
                b.param.copy_(torch.cat(parts))

    def _merge_touched(self) -> None:
        """A parameter counts as used if any rank produced a gradient for it (ranks can differ when a
        batch lacks a modality); one small all-reduce, only when some parameter was left untouched."""
        flags = [t for b in self.buffers for t in b.touched]
        if self.world == 1:
            return
        import torch.distributed as dist

        dev = self.buffers[0].device
        t = torch.tensor(flags, dtype=torch.float32).to(dev)
        if self.transport == "symm":
            t = self.symm.all_reduce_vector(t)
        else:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        merged = (t > 0).cpu().tolist()
        k = 0
        for b in self.buffers:
            n = len(b.touched)
            b.touched = merged[k:k + n]
            k += n

    def _global_norm_sq(self, shards: Optional[List[torch.Tensor]]) -> torch.Tensor:
        opt = self.optimizer
        if shards is None:
            return opt.local_grad_sumsq(shard_only=False)
        if self.transport == "symm":  # the reduce-scatter kernel already summed the squares of its shard
            opt.norm_sq.copy_(self.symm.local_sumsq)
            return self.symm.all_reduce_scalar(opt.norm_sq)
        opt.norm_sq.zero_()
        for g in shards:
            if g.is_cuda and g.dtype == torch.bfloat16:
                from ..ops import _ext

                _ext.get().sumsq_bf16(g, opt.norm_sq)
            else:
                opt.norm_sq += (g.float() ** 2).sum()
        import torch.distributed as dist

        dist.all_reduce(opt.norm_sq, op=dist.ReduceOp.SUM, group=self.group)
        return opt.norm_sq

    # ------------------------------------------------------------------ step
    def _on_touch(self, buf, i: int, kind: str) -> None:
        if not self._armed:
            return
        k = buf.index
        if not self._learned:
            self._order.setdefault(k, []).append((i, kind))
            return
        seen = self._seen.setdefault(k, set())
        seen.add(i)
        if kind == "accumulate" and self._trigger.get(k) == i and len(seen) == self._expected.get(k, -1) \
                and k not in self._early:
            self._early_reduce(k)

    def _early_reduce(self, k: int) -> None:
        dev = self.buffers[k].device
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=dev)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(dev))
        with torch.cuda.stream(self._comm_stream):
            self._comm_stream.wait_event(ev)
            self.symm.reduce_scatter_unit(k)
        self._early.add(k)

    def backward(self, loss: torch.Tensor) -> None:
        self._micro += 1
        overlap = self.overlap_reduce and self.transport == "symm"
        if overlap and self._micro == self.grad_accum:  # last micro-step: gradients become final
            self.symm.begin_step()
            self._step_begun = True
            self._armed = True
            self._seen = {}
            self._early = set()
        loss.backward()
        self._armed = False

    def optimizer_step(self, lr: float) -> torch.Tensor:
        """Reduce gradients, clip by global norm, update shards, refresh parameters, clear grads.
        Returns the squared global gradient norm *before* scaling by 1/(accum*world) (device)."""
        if self.check_touched:
            self._merge_touched()
        shards = self._reduce_scatter()
        norm_sq = self._global_norm_sq(shards)
        self.optimizer.step(lr=lr, norm_sq=norm_sq, grad_shards=shards)
        self._all_gather_params()
        self.optimizer.zero_grad()
        self._micro = 0
        self.last_norm_sq = norm_sq
        return norm_sq

    def grad_norm(self) -> torch.Tensor:
        """Global gradient norm of the last step in the units of the averaged gradient."""
        return self.last_norm_sq.sqrt() / float(self.grad_accum * self.world)

    # ------------------------------------------------------------------ state
    def optimizer_state(self) -> Dict:
        return {"opt": self.optimizer.state_dict(), "world": self.world, "rank": self.rank,
                "layout": [(b.name, b.numel, b.padded, list(zip(b.names, b.offsets))) for b in self.buffers]}

    def load_optimizer_state(self, sd: Dict) -> None:
        self.optimizer.load_state_dict(sd["opt"])

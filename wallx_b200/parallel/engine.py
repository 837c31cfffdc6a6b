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

Two parameter plans. Resident (default): every rank keeps all bf16 parameters, only the fp32 master
weights and Adam moments are sharded (ZeRO-1/2), and the updated shard is pushed to the peers after
AdamW. ``shard_params=True`` (ZeRO-3, the reference's ``FSDP2: True`` with ``reshard_after_forward``,
train_qact.py:42-49): the 2-D weights of every decoder layer and vision block are stored as rows per
rank (:mod:`wallx_b200.parallel.zero3`); on the NVLink transport the forward and dgrad GEMMs pull the
peers' rows inside the kernel, the wgrad GEMMs write a local bf16 gradient that each rank reduces for
its rows, and AdamW updates the owner's rows in place -- no all-gather or push of those weights exists
as a separate step.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

import contextlib

from ..train.optim import FlatAdamW
from .flat import FlatBuffer
from .zero3 import GatherWorkspace, RowShardedBuffer, zero3_units


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
                 master_dtype=torch.float32, symm=None, shard_params: bool = False):
        self.model = model
        self.world, self.rank = world, rank
        self.transport = transport if world > 1 else "local"
        self.group = group
        self.symm = symm
        self.grad_accum = grad_accum
        self.shard_params = bool(shard_params)
        pg = param_group_fn or (lambda name: ("default", 1.0, weight_decay))
        self.buffers: List[FlatBuffer] = []
        if self.shard_params:
            units = zero3_units(model, world)
        else:
            units = [(n, ps, "flat") for n, ps in default_units(model)]
        alloc = None
        align = FlatBuffer.ALIGN * world
        if self.transport == "symm" and symm is not None:
            p_total = g_total = 0
            for _, ps, kind in units:
                if kind == "rows":
                    a, b = RowShardedBuffer.sizes([p for _, p in ps], world)
                else:
                    a = b = (sum(p.numel() for _, p in ps) + align - 1) // align * align
                p_total += a
                g_total += b
            symm.reserve(p_total, dtype=units[0][1][0][1].dtype, grad_elems=g_total)
            alloc = (symm.alloc_param, symm.alloc_grad)
        row_mode = "gathered" if self.transport == "symm" else "materialized"
        for uname, ps, kind in units:
            groups = [pg(n) for n, _ in ps]
            if kind == "rows":
                self.buffers.append(RowShardedBuffer(ps, world, rank, groups, name=uname, alloc=alloc,
                                                     master_dtype=master_dtype, mode=row_mode))
            else:
                self.buffers.append(FlatBuffer(ps, world, rank, groups, name=uname, alloc=alloc, master_dtype=master_dtype))
        self.workspace = None
        rows_units = [b for b in self.buffers if b.kind == "rows" and b.mode == "gathered"]
        if rows_units:  # NVLink mode: two staging slots for the weight a GEMM is gathering (two for a dual-expert launch)
            dev = rows_units[0].device
            biggest = max(R * C for b in rows_units for R, C in b.shapes)
            self.workspace = GatherWorkspace(biggest, dev, slots=2, dtype=rows_units[0].dtype)
            self._ag_flags = torch.zeros(sum(b.flag_words() for b in rows_units), dtype=torch.int32, device=dev)
            ebytes = symm.param_arena.element_size()
            used = 0
            for b in rows_units:
                off = b.param.data_ptr() - symm.param_arena.data_ptr()
                assert off % ebytes == 0
                used += b.attach_gather([p + off for p in symm.param_ptrs], self.workspace, self._ag_flags[used:])
        self.optimizer = FlatAdamW(self.buffers, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                   max_grad_norm=max_grad_norm, grad_accum=grad_accum * world)
        if self.buffers and self.buffers[0].device.type == "cuda":
            # per-tile-shape GEMM rates of this device for the tile cost model (measured once per process, a few ms)
            from ..ops import _ext
            from ..ops import gemm as G

            import os

            if hasattr(_ext.get(), "gemm_tile_rates") and os.environ.get("WALLX_CALIBRATE", "1") != "0":
                G.calibrate_tile_rates(self.buffers[0].device)
        self.last_norm_sq: Optional[torch.Tensor] = None
        self.last_bad: Optional[torch.Tensor] = None  # device float: some rank's device-side wait ran out in the last step
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
                    self._trigger[k] = tuple(order[-1])
                self._learned = True
            return self.symm.grad_shards()
        import torch.distributed as dist

        shards = []
        for b in reversed(self.buffers):
            if b.kind == "rows":  # whole-gradient all-reduce, then this rank's rows of every weight
                tmp = b.grad if b.grad.is_cuda else b.grad.float()
                dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=self.group)
                out = torch.zeros(b.shard_size, device=b.device, dtype=b.grad.dtype)
                for goff, n, ooff in b.rs_segments():
                    out[ooff:ooff + n] = tmp[goff:goff + n].to(out.dtype)
                shards.append(out)
                continue
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
            if b.kind == "rows":  # materialized mode: refresh the whole parameters from the owners' rows
                with torch.no_grad():
                    for i, p in enumerate(b.params):
                        p.data.copy_(b.gather_full(i, self.group).to(p.dtype))
                continue
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
            bad = self._local_bad()
            if bad is None:
                opt.norm_sq.copy_(self.symm.local_sumsq)
                return self.symm.all_reduce_scalar(opt.norm_sq)
            # the same small all-reduce carries "a bounded wait ran out on some rank": every rank then sees a
            # non-finite norm, which makes the AdamW kernel skip the update on all ranks alike
            v = self.symm.all_reduce_vector(torch.cat([self.symm.local_sumsq.reshape(1), bad.reshape(1)]))
            self.last_bad = v[1:2]
            opt.norm_sq.copy_(torch.where(v[1:2] > 0, torch.full_like(v[0:1], float("nan")), v[0:1]))
            return opt.norm_sq
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
        # both kinds fire after the kernel that produces the gradient was enqueued on the current stream
        if self._trigger.get(k) == (i, kind) and len(seen) == self._expected.get(k, -1) and k not in self._early:
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

    def backward(self, loss: torch.Tensor, last: Optional[bool] = None) -> None:
        """Backward of one micro-batch. ``last`` says whether the optimizer step follows (its gradients are then
        final and units may be reduced while backward still runs); None = the ``grad_accum``-th micro-batch since the
        last step. A caller whose accumulation can end early (end of an epoch) passes it explicitly."""
        self._micro += 1
        overlap = self.overlap_reduce and self.transport == "symm"
        if last is None:
            last = self._micro == self.grad_accum
        if self._step_begun:
            # units were already reduced for this step and another backward arrives (the caller announced the last
            # micro-batch too early): their gradients change again, so every unit is reduced again after backward
            self._step_begun = False
            self._early = set()
        if overlap and last:
            self.symm.begin_step()
            self._step_begun = True
            self._armed = True
            self._seen = {}
            self._early = set()
        loss.backward()
        self._armed = False

    def _local_bad(self) -> Optional[torch.Tensor]:
        """Device float, 1.0 when one of this rank's bounded device-side waits ran out since the last host check
        (a peer stalled past the barrier limit, a GEMM gave up on an mbarrier or a gathered tile)."""
        dev = self.buffers[0].device
        if dev.type != "cuda":
            return None
        flags = []
        st = getattr(self.symm, "status", None) if self.symm is not None else None
        if st is not None:
            flags.append(st[:1] != 0)
        from ..ops import _ext

        C = _ext.get(required=False)
        if C is not None and hasattr(C, "status_tensor"):
            flags.append(C.status_tensor(dev.index or 0)[:1] != 0)
        if not flags:
            return None
        bad = flags[0]
        for f in flags[1:]:
            bad = bad | f
        return bad.float()

    def check_status(self) -> None:
        """Host check (synchronises): raise if any rank's device-side wait ran out in a step since the last check.
        Such a step was skipped on every rank (non-finite norm), so parameters are intact and ranks agree."""
        bad = self.last_bad
        if bad is not None and float(bad.item()) > 0:
            self.last_bad = None
            if self.symm is not None and hasattr(self.symm, "status"):
                self.symm.status.zero_()
            from ..ops import gemm as G

            try:
                G.check_status(self.buffers[0].device)
            except RuntimeError:
                pass
            raise RuntimeError("a device-side wait timed out on some rank (stalled or failed peer); the affected "
                               "optimizer step was skipped on every rank")

    def optimizer_step(self, lr: float) -> torch.Tensor:
        """Reduce gradients, clip by global norm, update shards, refresh parameters, clear grads.
        Returns the squared global gradient norm *before* scaling by 1/(accum*world) (device).
        The gradient is averaged over the micro-batches actually accumulated since the last step."""
        if self.check_touched:
            self._merge_touched()
        if self._micro > 0:
            self.optimizer.grad_accum = self._micro * self.world
        self._last_micro = self._micro or self.grad_accum
        shards = self._reduce_scatter()
        norm_sq = self._global_norm_sq(shards)
        if self.transport != "symm":
            bad = self._local_bad()
            if bad is not None:
                norm_sq.copy_(torch.where(bad > 0, torch.full_like(norm_sq, float("nan")), norm_sq))
                self.last_bad = bad
        self.optimizer.step(lr=lr, norm_sq=norm_sq, grad_shards=shards)
        self._all_gather_params()
        self.optimizer.zero_grad()
        self._micro = 0
        self._step_begun = False
        self.last_norm_sq = norm_sq
        return norm_sq

    def grad_norm(self) -> torch.Tensor:
        """Global gradient norm of the last step in the units of the averaged gradient."""
        return self.last_norm_sq.sqrt() / float(getattr(self, "_last_micro", self.grad_accum) * self.world)

    # ------------------------------------------------------------------ whole parameters of a sharded model
    @contextlib.contextmanager
    def gathered_parameters(self, writeback: bool = False):
        """Inside the block every row-sharded parameter holds its whole, current value (checkpoint export,
        ``state_dict()``, graph-captured inference). Collective: every rank must enter. With ``writeback`` the
        values found at exit (e.g. after ``load_state_dict``) replace the owners' rows and their fp32 masters, and
        the resident flat buffers' masters are refreshed too."""
        swapped = []
        for b in self.buffers:
            if b.kind != "rows":
                continue
            if b.mode == "gathered":
                for i, p in enumerate(b.params):
                    swapped.append((b, i, p, p.data))
                    p.data = b.gather_full(i, self.group)
            elif b.mode == "materialized" and not writeback:
                pass  # the whole parameters are kept current after every step
        try:
            yield self
        finally:
            with torch.no_grad():
                if writeback:
                    for b in self.buffers:
                        if b.kind == "rows":
                            for i, p in enumerate(b.params):
                                b.load_rows_from_full(i, p.data)
                for b, i, p, old in swapped:
                    p.data = old
                if writeback:
                    self.refresh_master()

    def close(self) -> None:
        """Detach the engine from the model (hooks, gradient sinks, gather records) so that both can be freed."""
        for b in self.buffers:
            b.release()
        self.buffers = []
        self.optimizer.buffers = []
        self.workspace = None
        self.symm = None

    def refresh_master(self) -> None:
        """fp32 master shards := current bf16 parameter shards (after loading weights into the model)."""
        for b in self.buffers:
            s0, s1 = b.shard_range
            b.master.copy_(b.param[s0:s1].to(b.master.dtype))

    # ------------------------------------------------------------------ state
    def optimizer_state(self) -> Dict:
        layout = []
        for b in self.buffers:
            if b.kind == "rows":
                layout.append((b.name, b.numel, b.shard_size, list(zip(b.names, b.offsets)), "rows", list(b.shapes)))
            else:
                layout.append((b.name, b.numel, b.padded, list(zip(b.names, b.offsets)), "flat",
                               [tuple(p.shape) for p in b.params]))
        return {"opt": self.optimizer.state_dict(), "world": self.world, "rank": self.rank, "layout": layout}

    def load_optimizer_state(self, sd: Dict) -> None:
        self.optimizer.load_state_dict(sd["opt"])

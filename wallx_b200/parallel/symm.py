"""Symmetric-memory transport: peer pointers over NVLink / NVSwitch + hand-written collectives.

Bootstrap (allocation, handle exchange, peer pointer tables) uses
``torch.distributed._symmetric_memory``; the data plane is this package's kernels
(``csrc/comm.cu``): a flag barrier with bounded waits, a one-shot reduce-scatter that pulls every
peer's gradient shard and sums in fp32, a one-shot all-gather that pushes the updated bf16 shard
into every peer's resident parameters, and a small-vector all-reduce for the gradient norm and
logged scalars. No NCCL call is made on these paths (NCCL only serves the bootstrap rendezvous).

Reference parity: the NCCL collectives that accelerate / torch FSDP2 issue for the reference trainer
(train_qact.py:42-49; wall_x/trainer/qwen_vl_act_trainer.py:335-337 grad-norm all-reduce, :352-423 scalar gathers).

Two bf16 arenas (parameters, gradients) are allocated once; every :class:`FlatBuffer` is a view, so
one rendezvous covers the whole model.
"""
from __future__ import annotations

from typing import List

import torch

from ..ops import _ext

MAX_VEC = 4096  # floats per rank in the small all-reduce scratch
FLAG_WORDS = 8 * 256  # int32 flag slots: 8 for the global barrier, then 8 per unit (up to 255 units)


class SymmComm:
    def __init__(self, group, device, barrier_timeout_s: float = 30.0):
        """``barrier_timeout_s`` bounds every wait on a peer (clamped to 10 min by the kernel). Ranks are not
        synchronised by the host, so the limit has to cover the longest time one rank may lag behind another
        between two barriers (a data-loader stall, a first-step lazy initialisation), not just network latency."""
        import torch.distributed as dist

        self.timeout_ms = max(1, int(barrier_timeout_s * 1000))
        # multimem stores for the parameter push when the fabric offers a multicast mapping (WALLX_NVLS=0 turns it off:
        # tests in which a rank may die keep every multicast object out of the picture)
        import os

        self.use_multicast = os.environ.get("WALLX_NVLS", "1") != "0"
        self.param_mc = 0
        import torch.distributed._symmetric_memory as symm_mem

        self.symm_mem = symm_mem
        self.group = group
        self.device = device
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("symmetric transport supports up to 8 ranks of one NVSwitch domain")
        # control block: [0, FLAG_WORDS) int32 flags | then world * MAX_VEC floats of scratch
        self.ctrl = symm_mem.empty(FLAG_WORDS + self.world * MAX_VEC, dtype=torch.float32, device=device)
        self.ctrl.zero_()
        self.ctrl_hdl = symm_mem.rendezvous(self.ctrl, group)
        base = [int(p) for p in self.ctrl_hdl.buffer_ptrs]
        self.flag_ptrs = base
        self.scratch_ptrs = [p + FLAG_WORDS * 4 for p in base]
        self.scratch = self.ctrl[FLAG_WORDS:]
        self.unit_step = 0
        self.epoch = 0
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.param_arena = self.grad_arena = None
        self._cursor = {"param": 0, "grad": 0}
        self.local_sumsq = torch.zeros(1, dtype=torch.float32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)

    # ------------------------------------------------------------------ allocation
    def reserve(self, total_elems: int, dtype=torch.bfloat16, grad_elems: int = 0) -> None:
        """Allocate the two arenas. With row-sharded parameters the parameter arena holds shards and the gradient
        arena whole gradients, so their sizes differ (``grad_elems``)."""
        sm = self.symm_mem
        grad_elems = grad_elems or total_elems
        # symmetric allocations are not returned to the caching allocator, so an engine that replaces another one
        # (same transport object) takes over the arenas when they are large enough
        if self.param_arena is None or self.param_arena.numel() < total_elems or self.param_arena.dtype != dtype:
            self.param_arena = None
            self.param_arena = sm.empty(total_elems, dtype=dtype, device=self.device)
            hdl = sm.rendezvous(self.param_arena, self.group)
            self.param_ptrs = [int(p) for p in hdl.buffer_ptrs]
            # NVSwitch multicast mapping of the arena (0 when the fabric has none): lets the parameter push leave
            # this GPU once instead of once per peer
            self.param_mc = int(getattr(hdl, "multicast_ptr", 0) or 0) if self.use_multicast else 0
        if self.grad_arena is None or self.grad_arena.numel() < grad_elems or self.grad_arena.dtype != dtype:
            self.grad_arena = None
            self.grad_arena = sm.empty(grad_elems, dtype=dtype, device=self.device)
            self.grad_ptrs = [int(p) for p in sm.rendezvous(self.grad_arena, self.group).buffer_ptrs]
        self.param_arena.zero_()
        self.grad_arena.zero_()
        self._cursor = {"param": 0, "grad": 0}

    def _take(self, which: str, n: int, dtype) -> torch.Tensor:
        arena = self.param_arena if which == "param" else self.grad_arena
        if arena is None:
            raise RuntimeError("SymmComm.reserve() must be called before allocating flat buffers")
        assert arena.dtype == dtype, "arena dtype mismatch"
        c = self._cursor[which]
        if c + n > arena.numel():
            raise RuntimeError("symmetric arena exhausted")
        self._cursor[which] = c + n
        return arena[c:c + n]

    def alloc_param(self, n: int, dtype) -> torch.Tensor:
        return self._take("param", n, dtype)

    def alloc_grad(self, n: int, dtype) -> torch.Tensor:
        return self._take("grad", n, dtype)

    def arena_bytes(self) -> int:
        """Bytes of the two symmetric arenas that the current engine uses (they are not part of the caching
        allocator's statistics)."""
        if self.param_arena is None:
            return 0
        e = self.param_arena.element_size()
        return (self._cursor["param"] + self._cursor["grad"]) * e

    def register_buffers(self, buffers) -> None:
        """Build the device tables: per unit the pieces of the gradient arena this rank reduces (one for a flat
        buffer, one per weight for a row-sharded unit) and the pieces of the parameter arena it pushes to its peers
        (none for row-sharded units: their rows are read in place by the peers' GEMMs)."""
        rows, push, out_off = [], [], 0
        elem = self.param_arena.element_size()
        pbase, gbase = self.param_arena.data_ptr(), self.grad_arena.data_ptr()
        self.views, self.unit_rows = [], []
        for b in buffers:
            g0 = (b.grad.data_ptr() - gbase) // elem
            p0 = (b.param.data_ptr() - pbase) // elem
            first = len(rows)
            for goff, n, ooff in b.rs_segments():
                rows.append([g0 + goff, n, out_off + ooff])
            self.unit_rows.append((first, len(rows)))
            for poff, n in b.push_segments():
                push.append([p0 + poff, n, 0])
            self.views.append((out_off, b.shard_size))
            out_off += b.shard_size
        self.table = torch.tensor(rows, dtype=torch.int64, device=self.device).reshape(-1, 3)
        self.push_table = torch.tensor(push, dtype=torch.int64, device=self.device).reshape(-1, 3)
        self.gshard = torch.zeros(out_off, dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------ collectives
    def barrier(self) -> None:
        self.epoch += 1
        _ext.get().symm_barrier(self.flag_ptrs, self.rank, self.epoch, self.status, self.timeout_ms)

    def check(self) -> None:
        """Raise if a barrier wait ran out (a peer died or stalled); synchronises."""
        st = int(self.status[0].item())
        if st != 0:
            self.status.zero_()
            raise RuntimeError(f"symmetric barrier timed out waiting for rank {st - 16}")

    def reduce_scatter_grads(self, buffers) -> List[torch.Tensor]:
        C = _ext.get()
        self.barrier()  # every rank has finished writing its gradients
        self.local_sumsq.zero_()
        C.rs_reduce(self.grad_ptrs, self.table, self.gshard, self.local_sumsq)
        return [self.gshard[o:o + n] for o, n in self.views]

    # Per-unit variant: every unit has its own flag slots, so the ranks may reach the units at
    # different times and in any order (one rank can reduce a unit while backward still runs, another
    # after it) without the barriers of different units getting mixed up.
    def begin_step(self) -> None:
        self.unit_step += 1
        self.local_sumsq.zero_()

    def reduce_scatter_unit(self, k: int) -> None:
        """Barrier on unit k's flags, then pull and sum unit k's gradient shard (current stream)."""
        if 8 * (k + 2) > FLAG_WORDS:
            raise ValueError("too many units for the per-unit flag block")
        C = _ext.get()
        C.symm_barrier([p + 32 * (k + 1) for p in self.flag_ptrs], self.rank, self.unit_step, self.status, self.timeout_ms)
        a, b = self.unit_rows[k]
        C.rs_reduce(self.grad_ptrs, self.table[a:b], self.gshard, self.local_sumsq)

    def grad_shards(self) -> List[torch.Tensor]:
        return [self.gshard[o:o + n] for o, n in self.views]

    def all_reduce_vector(self, t: torch.Tensor) -> torch.Tensor:
        C = _ext.get()
        v = t.detach().float().contiguous().reshape(-1)
        if v.numel() > MAX_VEC:
            raise ValueError(f"small all-reduce handles at most {MAX_VEC} floats")
        C.small_allreduce_write(self.scratch_ptrs, v, self.rank)
        self.barrier()
        out = torch.empty_like(v)
        C.small_allreduce_sum(self.scratch, out, self.world)
        self.barrier()  # nobody overwrites the scratch before everyone has read it
        return out.reshape(t.shape)

    def all_reduce_scalar(self, t: torch.Tensor) -> torch.Tensor:
        t.copy_(self.all_reduce_vector(t))
        return t

    def all_gather_params(self, buffers) -> None:
        if self.push_table.shape[0] > 0:
            if self.param_mc:
                _ext.get().ag_push_multicast(self.param_mc, self.param_ptrs[self.rank], self.push_table)
            else:
                _ext.get().ag_push(self.param_ptrs, self.push_table, self.rank)
        # all pushes have landed, and every owner has updated its rows, before anyone reads the parameters
        self.barrier()

"""Row-sharded parameter storage (ZeRO-3 / FSDP): every 2-D weight of a unit lives as ``rows / world`` rows per rank.

This is the storage side of the reference's recommended mode, torch FSDP2 with ``reshard_after_forward=True``
(train_qact.py:42-49, workspace/lerobot_example/config_qact.yml ``FSDP2: True``; shard units =
``_no_split_modules``, modeling_qwen2_5_vl_act.py:745). The compute side differs by design: nothing ever runs a
stand-alone all-gather of a unit. On the NVLink transport a weight's rows are pulled from the peers *inside* the GEMM
that consumes it (``csrc/gemm.cu``, ``gemm_ag_launch``: forward and dgrad), into a staging buffer that the next GEMM
reuses, so the full parameter never persists ("reshard after forward" for free). The weight gradient is formed
locally by the wgrad GEMM in a bf16 buffer and each rank reduces *its rows* with the peer-load reduce-scatter kernel;
AdamW then updates the owner's rows in place, so no parameter push follows the optimizer in this mode.

Three modes of one layout:

``local``         one rank: the shard is the whole weight and the parameters view it (no gather at all).
``materialized``  ``torch.distributed`` transport (gloo on CPU, NCCL): the full parameter stays allocated and is
                  refreshed from the shards by a collective after each optimizer step (plain baseline and the
                  CPU test path of the shard arithmetic).
``gathered``      NVLink transport: ``p.data`` is a view of a shared staging slot, filled by the consuming GEMM.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .flat import FlatBuffer, ParamSegment, _round_up


def shardable(p: torch.Tensor, world: int) -> bool:
    """Rows split evenly and every row is a whole number of 16-byte units (bulk copies, TMA)."""
    return p.dim() == 2 and p.shape[0] % world == 0 and p.shape[1] % 8 == 0 and p.shape[0] // world >= 1


class GatherWorkspace:
    """Local staging memory shared by all sharded weights of a model (one weight at a time per slot)."""

    def __init__(self, max_elems: int, device, slots: int = 2, dtype=torch.bfloat16):
        self.buf = torch.empty(slots, max_elems, dtype=dtype, device=device)
        self.max_elems = int(max_elems)
        self.slots = slots
        # which weight was gathered into each slot last (set whenever a gather into the slot is enqueued): a launch
        # may read a slot as a plain operand only while the weight it wants is still the owner
        self.owner = [None] * slots

    def view(self, rows: int, cols: int, slot: int = 0) -> torch.Tensor:
        n = rows * cols
        if n > self.max_elems:
            raise ValueError(f"gather workspace holds {self.max_elems} elements, weight needs {n}")
        return self.buf[slot, :n].view(rows, cols)


class GatheredWeight:
    """What the fused-gather GEMM needs to know about one row-sharded weight: the peers' shard addresses, the
    per-tile ready flags with their epoch, and the staging view the GEMM reads the whole weight from."""

    def __init__(self, rows: int, cols: int, world: int, rank: int, peer_ptrs: Sequence[int], flags: torch.Tensor,
                 staging: torch.Tensor, slot: int = 0):
        self.rows, self.cols, self.world, self.rank = int(rows), int(cols), int(world), int(rank)
        self.rows_per_rank = self.rows // self.world
        self.peer_ptrs = [int(p) for p in peer_ptrs]
        self.flags = flags
        self.epoch = 0
        self.slot = int(slot)
        self._staging = staging
        self.workspace: Optional[GatherWorkspace] = None  # set by the engine: slot ownership for prefetched gathers
        self.prefetched = False  # whole and current in its staging view, gathered ahead of its use
        self.n_pullers: Optional[int] = None  # fixed by the first launch: the flags count arrivals of that many copy CTAs

    def staging(self, slot: Optional[int] = None) -> torch.Tensor:
        return self._staging

    def next_epoch(self) -> int:
        """Called once per enqueued gather of this weight (fused into a GEMM or carried by another launch)."""
        self.epoch += 1
        if self.epoch >= (1 << 24):  # flags are int32 counts of n_pullers * epoch
            self.flags.zero_()
            self.epoch = 1
        self.prefetched = False
        ws = self.workspace
        if ws is not None:
            prev = ws.owner[self.slot]
            if prev is not None and prev is not self:
                prev.prefetched = False  # its copy in the slot is about to be overwritten
            ws.owner[self.slot] = self
        return self.epoch

    def in_place(self) -> bool:
        """True when the whole, current weight sits in its staging view because an earlier launch gathered it ahead
        of time and nothing has been gathered into that slot since."""
        ws = self.workspace
        return bool(self.prefetched and ws is not None and ws.owner[self.slot] is self)

    def pin_pullers(self, n_pullers: int) -> None:
        """The ready flags count ``n_pullers`` arrivals per launch, so the number must not change while counts from
        earlier launches are still in the flags."""
        if self.n_pullers is None:
            self.n_pullers = int(n_pullers)
        elif self.n_pullers != int(n_pullers):
            self.flags.zero_()
            self.epoch = 0
            self.n_pullers = int(n_pullers)


def slot_of(name: str) -> int:
    """Staging slot of a weight. Weights that are gathered by one launch must sit in different slots: the two experts'
    gate/up (and down) projections, and the QKV and output projections of a block's attention (their gathers ride
    together on the FFN's weight-gradient GEMM in backward)."""
    return 1 if (".experts.1." in name or "qkv" in name) else 0


class RowShardedBuffer:
    """The 2-D weights of one unit, split by rows over the ranks, with this rank's optimizer state.

    Duck-types :class:`FlatBuffer` for the optimizer and the engine: ``param`` is this rank's bf16 shard (the
    concatenation of its rows of every weight), ``grad`` the *whole* bf16 gradient of the unit (written by the wgrad
    GEMMs), ``shard_range`` covers all of ``param``, ``offsets`` are shard-local.
    """

    ALIGN = FlatBuffer.ALIGN
    kind = "rows"

    @staticmethod
    def sizes(params: Sequence[torch.Tensor], world: int) -> Tuple[int, int]:
        """``(shard elements, whole-gradient elements)`` including alignment padding."""
        shard = sum(p.numel() // world for p in params)
        full = sum(p.numel() for p in params)
        if world == 1:
            n = _round_up(full, RowShardedBuffer.ALIGN)
            return n, n
        return _round_up(shard, RowShardedBuffer.ALIGN), _round_up(full, RowShardedBuffer.ALIGN * world)

    def __init__(self, named_params: Sequence[Tuple[str, nn.Parameter]], world: int = 1, rank: int = 0,
                 groups: Optional[Sequence[Tuple[str, float, float]]] = None, name: str = "", alloc=None,
                 master_dtype=torch.float32, mode: str = "materialized"):
        assert len(named_params) > 0
        if world == 1:
            mode = "local"
        assert mode in ("local", "materialized", "gathered")
        self.name, self.mode = name, mode
        self.world, self.rank = world, rank
        p0 = named_params[0][1]
        self.device, self.dtype = p0.device, p0.dtype
        if groups is None:
            groups = [("default", 1.0, 0.0)] * len(named_params)
        order = sorted(range(len(named_params)), key=lambda i: (groups[i][0], i))
        self.names: List[str] = []
        self.params: List[nn.Parameter] = []
        self.offsets: List[int] = []       # shard-local element offset of each weight's rows
        self.grad_offsets: List[int] = []  # element offset of each whole weight in ``grad``
        self.shapes: List[Tuple[int, int]] = []
        self.segments: List[ParamSegment] = []
        off = goff = 0
        for i in order:
            n, p = named_params[i]
            if not shardable(p, world):
                raise ValueError(f"{n}: shape {tuple(p.shape)} cannot be split by rows over {world} ranks")
            g = groups[i]
            if not self.segments or self.segments[-1].name != g[0]:
                self.segments.append(ParamSegment(off, off, g[1], g[2], g[0]))
            self.names.append(n)
            self.params.append(p)
            self.offsets.append(off)
            self.grad_offsets.append(goff)
            self.shapes.append((int(p.shape[0]), int(p.shape[1])))
            off += p.numel() // world
            goff += p.numel()
            self.segments[-1].end = off
        self.numel = goff            # logical parameters of the unit
        self.shard_numel = off
        self.shard_size, self.padded = self.sizes([p for p in self.params], world)
        default = lambda n, dtype: torch.zeros(n, device=self.device, dtype=dtype)
        alloc_param, alloc_grad = alloc if alloc is not None else (default, default)
        self.param = alloc_param(self.shard_size, self.dtype)
        self.grad = alloc_grad(self.padded, self.dtype)
        self.shard_range = (0, self.shard_size)
        with torch.no_grad():
            for p, o, go, (R, C) in zip(self.params, self.offsets, self.grad_offsets, self.shapes):
                rr = R // world
                self.param[o:o + rr * C].copy_(p.data[rank * rr:(rank + 1) * rr].reshape(-1))
                if mode == "local":
                    p.data = self.param[o:o + R * C].view(R, C)
                p.grad = self.grad[go:go + R * C].view(R, C)
        self.touched = [False] * len(self.params)
        self._hook_handles = []
        self.on_touch = None
        for i, p in enumerate(self.params):
            self._hook_handles.append(p.register_post_accumulate_grad_hook(self._make_hook(i, "accumulate")))
        if self.param.is_cuda:  # weight-gradient GEMMs add straight into the unit's gradient buffer
            from ..ops import functional as F_

            for i, (p, go, (R, C)) in enumerate(zip(self.params, self.grad_offsets, self.shapes)):
                F_.register_grad_sink(p, self.grad[go:go + R * C].view(R, C), self._make_hook(i, "sink"))
        self.seg_of_param = []
        for o in self.offsets:
            self.seg_of_param.append(next(k for k, sg in enumerate(self.segments) if sg.start <= o < sg.end))
        self.master = self.param.to(master_dtype).clone()
        self.exp_avg = torch.zeros(self.shard_size, device=self.device, dtype=master_dtype)
        self.exp_avg_sq = torch.zeros(self.shard_size, device=self.device, dtype=master_dtype)
        self.gathered: List[Optional[GatheredWeight]] = [None] * len(self.params)

    # ------------------------------------------------------------------ hooks / bookkeeping (as FlatBuffer)
    def _make_hook(self, i: int, kind: str = "accumulate"):
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

    def rows_per_rank(self, i: int) -> int:
        return self.shapes[i][0] // self.world

    def shard_len(self, i: int) -> int:
        return self.rows_per_rank(i) * self.shapes[i][1]

    def update_ranges(self, touched=None) -> List[Tuple[int, int, ParamSegment]]:
        touched = self.touched if touched is None else touched
        if all(touched):
            return self.shard_segments()
        out: List[Tuple[int, int, ParamSegment]] = []
        for i, o in enumerate(self.offsets):
            if not touched[i]:
                continue
            lo, hi = o, o + self.shard_len(i)
            seg = self.segments[self.seg_of_param[i]]
            if out and out[-1][1] == lo and out[-1][2] is seg:
                out[-1] = (out[-1][0], hi, seg)
            else:
                out.append((lo, hi, seg))
        return out

    def shard_segments(self) -> List[Tuple[int, int, ParamSegment]]:
        out = []
        for k, seg in enumerate(self.segments):
            hi = seg.end if k + 1 < len(self.segments) else self.shard_size
            if hi > seg.start:
                out.append((seg.start, hi, seg))
        return out

    def rebind_grads(self) -> None:
        for p, go, (R, C) in zip(self.params, self.grad_offsets, self.shapes):
            p.grad = self.grad[go:go + R * C].view(R, C)

    def zero_grad(self) -> None:
        self.grad.zero_()

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {"master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq}

    # ------------------------------------------------------------------ transport tables
    def rs_segments(self) -> List[Tuple[int, int, int]]:
        """``(offset in the whole gradient, length, offset in the shard)`` of the pieces this rank reduces."""
        return [(go + self.rank * self.shard_len(i), self.shard_len(i), o)
                for i, (o, go) in enumerate(zip(self.offsets, self.grad_offsets))]

    def push_segments(self) -> List[Tuple[int, int]]:
        return []  # the owner's rows are read in place by the peers' GEMMs

    # ------------------------------------------------------------------ gather plumbing
    def attach_gather(self, peer_param_ptrs: Sequence[int], workspace: GatherWorkspace, flags: torch.Tensor) -> int:
        """NVLink mode: point every parameter at its staging slot and record where the peers keep their rows.
        ``peer_param_ptrs[r]`` is the address of rank r's copy of ``self.param``; ``flags`` is an int32 tensor with
        at least :meth:`flag_words` entries. Returns the number of flag words used."""
        assert self.mode == "gathered"
        used = 0
        esize = self.param.element_size()
        for i, (p, o, (R, C), n) in enumerate(zip(self.params, self.offsets, self.shapes, self.names)):
            slot = slot_of(n) % workspace.slots
            nf = (R + 255) // 256
            gw = GatheredWeight(R, C, self.world, self.rank, [b + o * esize for b in peer_param_ptrs],
                                flags[used:used + nf], workspace.view(R, C, slot), slot)
            used += nf
            gw.workspace = workspace
            self.gathered[i] = gw
            p.data = gw.staging()
            p._wx_shard = gw
        return used

    def flag_words(self) -> int:
        return sum((R + 255) // 256 for R, _ in self.shapes)

    def own_rows(self, i: int) -> torch.Tensor:
        """This rank's rows of weight i as a ``[rows / world, cols]`` view of the shard."""
        o, (R, C) = self.offsets[i], self.shapes[i]
        rr = R // self.world
        return self.param[o:o + rr * C].view(rr, C)

    def load_rows_from_full(self, i: int, full: torch.Tensor) -> None:
        rr = self.rows_per_rank(i)
        self.own_rows(i).copy_(full[self.rank * rr:(self.rank + 1) * rr].to(self.param.dtype))

    def gather_full(self, i: int, group=None) -> torch.Tensor:
        """Whole weight i by a plain collective (checkpoints, inference on a sharded model, tests)."""
        R, C = self.shapes[i]
        if self.world == 1:
            return self.own_rows(i).clone()
        import torch.distributed as dist

        mine = self.own_rows(i).contiguous()
        if mine.is_cuda:
            full = torch.empty(R, C, dtype=mine.dtype, device=mine.device)
            dist.all_gather_into_tensor(full, mine, group=group)
            return full
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=group)
        return torch.cat(parts, dim=0)


def zero3_units(model: nn.Module, world: int):
    """Units of the sharded mode: per vision block / decoder layer its row-shardable 2-D weights (``"rows"`` units),
    and one resident root unit with everything else (embeddings, head, norms, biases, action head): the small
    parameters are a few MB in total and every rank needs them whole in every layer."""
    claimed = set()
    units = []

    def take(prefix: str, mod: nn.Module):
        ps = [(f"{prefix}.{n}", p) for n, p in mod.named_parameters()
              if p.requires_grad and id(p) not in claimed and shardable(p, world)]
        for _, p in ps:
            claimed.add(id(p))
        if ps:
            units.append((prefix, ps, "rows"))

    visual = getattr(model, "visual", None)
    if visual is not None and hasattr(visual, "blocks"):
        for i, blk in enumerate(visual.blocks):
            take(f"visual.blocks.{i}", blk)
    lm = getattr(model, "model", None)
    if lm is not None and hasattr(lm, "layers"):
        for i, layer in enumerate(lm.layers):
            take(f"model.layers.{i}", layer)
    rest = [(n, p) for n, p in model.named_parameters() if p.requires_grad and id(p) not in claimed]
    if rest:
        units.append(("root", rest, "flat"))
    return units

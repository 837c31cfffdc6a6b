"""Weights whose all-gather is fused into the consuming GEMM (the compute side of ZeRO-3 style sharding).

A row-sharded weight keeps ``rows / world`` rows of a ``[rows, cols]`` bf16 weight per rank in symmetric
(peer-mapped) memory. :func:`ag_launch` multiplies by the whole weight without ever running a separate all-gather:
a few CTAs of the persistent tcgen05 GEMM grid pull the peers' rows over NVLink into a local staging buffer, tile by
tile, while the remaining CTAs multiply the tiles that have already arrived (``csrc/gemm.cu``, ``gemm_ag_launch``).
The backward pass gathers again for ``dx = dy @ W`` (MN-major weight operand, flags per 256 contraction rows).

The training engine uses this through :mod:`wallx_b200.parallel.zero3` (``TrainEngine(shard_params=True)``): every
GEMM of :mod:`wallx_b200.ops.functional` whose weight carries a gather record goes through :func:`ag_launch`, the
weight gradient is formed locally in bf16 and reduce-scattered by the peer-load kernel of ``csrc/comm.cu``.
:class:`ShardedWeight` is the stand-alone form (its own symmetric allocation) used by the kernel benchmarks and tests.

Reference parity: the reference shards parameters with torch FSDP2 through accelerate
(workspace/lerobot_example/config_qact.yml ``FSDP2: True``; train_qact.py:42-70), i.e. an NCCL all-gather followed by
cuBLAS; this is the fused equivalent. :func:`ag_dual_gate_up` is the same for the two FFN experts' gate/up projections
in one launch (wall_x/model/qwen2_5_based/modeling_qwen2_5_vl_act.py:228-330, csrc/dual_asym_grouped_gemm.cu:49-136).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..ops import _ext
from ..ops import gemm as G
from .zero3 import GatheredWeight, GatherWorkspace

import os as _os

# Copy CTAs per launch (of 148 SMs); fixed per weight because the ready flags count their arrivals. Every copy CTA keeps
# ten 16 KB bulk loads in flight (about 60 GB/s each over NVLink), and a layer's GEMMs need roughly 100 GB/s of remote
# weight traffic to stay fed, so a handful suffices; each one is an SM the multiplication does not get.
DEFAULT_PULLERS = int(_os.environ.get("WALLX_AG_PULLERS", "8"))
_PULLERS_FROM_ENV = "WALLX_AG_PULLERS" in _os.environ


STANDALONE_PULLERS = 16


def auto_pullers(specs: Sequence[G.GemmSpec], weights: Sequence[GatheredWeight]) -> int:
    """Copy CTAs for a launch. Weights of a training engine take the default (8: measured best inside the step, where
    most backward gathers ride on the weight-gradient GEMMs and every copy CTA is an SM the multiplication does not
    get). A stand-alone :class:`ShardedWeight` has nothing else to hide its gather behind: at least 16 (measured on the
    dual-expert FFN at 2K-32K tokens: 16 beat 8 and 14 everywhere), more when the multiplication is too short for the
    remote rows to arrive within it at about 30 GB/s per copy CTA, at most 32."""
    if not all(isinstance(w, ShardedWeight) for w in weights):
        return DEFAULT_PULLERS
    flops = sum(2.0 * s.M * s.N * s.K for s in specs)
    remote = sum(2.0 * w.rows * w.cols * (w.world - 1) / max(w.world, 1) for w in weights)
    t = max(flops / 1.2e15, 1e-6)
    n = int(-(-remote // (t * 30e9)))
    n = max(STANDALONE_PULLERS, min(32, n))
    return (n + 1) & ~1


class ShardedWeight(GatheredWeight):
    """``rows / world`` rows of a ``[rows, cols]`` bf16 weight in its own symmetric allocation, plus peer addresses."""

    def __init__(self, rows: int, cols: int, group, device, workspace: Optional[GatherWorkspace] = None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        if rows % world:
            raise ValueError(f"weight rows {rows} must divide evenly over {world} ranks")
        if cols % 8:
            raise ValueError("weight row length must be a multiple of 8 elements (16 bytes)")
        self.group = group
        if torch.device(device).type == "cpu":
            # CPU stand-in (tests of the shard arithmetic over gloo): same row split, the gather is a collective
            super().__init__(rows, cols, world, rank, [], None, None)
            self.shard = torch.zeros(self.rows_per_rank, cols, dtype=torch.float32)
            self.workspace = None
            return
        self.shard = symm_mem.empty(rows // world, cols, dtype=torch.bfloat16, device=device)
        self.shard.zero_()
        hdl = symm_mem.rendezvous(self.shard, group)
        flags = torch.zeros((rows + 255) // 256, dtype=torch.int32, device=device)
        super().__init__(rows, cols, world, rank, [int(p) for p in hdl.buffer_ptrs], flags, None)
        self.workspace = workspace if workspace is not None else GatherWorkspace(rows * cols, device, slots=1)

    def load_full(self, full: torch.Tensor) -> None:
        """Keep this rank's rows of a replicated full weight."""
        r0 = self.rank * self.rows_per_rank
        self.shard.copy_(full[r0:r0 + self.rows_per_rank].to(self.shard.dtype))

    def gather_full(self) -> torch.Tensor:
        """The whole weight by a plain collective (CPU stand-in and debugging; the GPU path never materialises it
        outside the GEMM's staging buffer)."""
        import torch.distributed as dist

        parts = [torch.empty_like(self.shard) for _ in range(self.world)]
        dist.all_gather(parts, self.shard.contiguous(), group=self.group)
        return torch.cat(parts, dim=0)

    def staging(self, slot: Optional[int] = None) -> torch.Tensor:
        self.slot = int(slot or 0)
        return self.workspace.view(self.rows, self.cols, self.slot)


def ag_launch(specs: Sequence[G.GemmSpec], weights: Sequence[GatheredWeight], n_pullers: int = 0) -> None:
    """One launch of one or two problems; ``specs[i].b`` must be weight i's staging view (distinct slots)."""
    if n_pullers:
        np_ = int(n_pullers)
    elif weights[0].n_pullers:
        np_ = weights[0].n_pullers  # fixed by the weight's first launch
    else:
        np_ = DEFAULT_PULLERS if _PULLERS_FROM_ENV else auto_pullers(specs, weights)
    for w in weights:
        w.pin_pullers(np_)
    _ext.get().gemm_ag([s.as_tuple() for s in specs], [w.peer_ptrs for w in weights], [w.flags for w in weights],
                       weights[0].rank, [w.rows_per_rank for w in weights], np_,
                       [w.next_epoch() for w in weights])


def ag_gemm(x: torch.Tensor, w: ShardedWeight, *, transpose_w: bool = False, bias=None, residual=None, flags: int = 0,
            out: Optional[torch.Tensor] = None, n_pullers: int = 0) -> torch.Tensor:
    """``x @ W.T`` (``transpose_w=False``, x ``[M, cols]``) or ``x @ W`` (``True``, x ``[M, rows]``)."""
    if not x.is_cuda:  # CPU stand-in: gather by collective, then the oracle's matmul and epilogue
        full = w.gather_full().to(torch.float32)
        y = x.float() @ (full if transpose_w else full.t())
        if bias is not None:
            y = y + bias.float()
        if flags & G.ACT_SWIGLU:
            from ..ops import ref

            y = ref.swiglu_interleaved(y)
        if residual is not None:
            y = y + residual.float()
        y = y.to(torch.float32 if (flags & G.OUT_FP32) else x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    M = x.shape[0]
    N = w.cols if transpose_w else w.rows
    if out is None:
        width = N // 2 if (flags & G.ACT_SWIGLU) else N
        out = torch.empty(M, width, device=x.device, dtype=torch.float32 if (flags & G.OUT_FP32) else torch.bfloat16)
    spec = G.GemmSpec(x, w.staging(), out, b_mn=transpose_w, bias=bias, residual=residual, flags=flags)
    ag_launch([spec], [w], n_pullers)
    return out


def ag_dual_gate_up(xs: Sequence[torch.Tensor], ws: Sequence[ShardedWeight], *, dyn: Sequence[Optional[torch.Tensor]] = (None, None),
                    m0: Sequence[int] = (0, 0), Ms: Sequence[Optional[int]] = (None, None),
                    outs: Optional[Sequence[torch.Tensor]] = None, n_pullers: int = 0) -> List[torch.Tensor]:
    """Both experts' ``silu(x Wg.T) * (x Wu.T)`` in one launch, with both interleaved gate/up weights gathered
    inside it. ``xs[i]`` is expert i's activations ``[*, hidden]`` (the same packed tensor with ``m0`` / ``Ms`` /
    ``dyn`` selecting each expert's segment, or two separate tensors); ``ws[i].rows`` is twice expert i's FFN width."""
    res = []
    specs = []
    for i, (x, w) in enumerate(zip(xs, ws)):
        M = Ms[i] if Ms[i] is not None else x.shape[0] - m0[i]
        out = outs[i] if outs is not None else torch.empty(x.shape[0], w.rows // 2, dtype=torch.bfloat16, device=x.device)
        specs.append(G.GemmSpec(x, w.staging(slot=i), out, M=M, m0=m0[i], dyn=dyn[i], flags=G.ACT_SWIGLU))
        res.append(out)
    ag_launch(specs, list(ws), n_pullers)
    return res

"""Sharded weights whose all-gather is fused into the consuming GEMM (ZeRO-3 style parameters).

A :class:`ShardedWeight` keeps ``rows / world`` rows of a ``[rows, cols]`` bf16 weight per rank in
symmetric (peer-mapped) memory. :func:`ag_linear` multiplies by the whole weight without ever
running a separate all-gather: a few CTAs of the persistent tcgen05 GEMM grid pull the peers'
shards over NVLink into a local staging buffer, tile by tile, while the remaining CTAs multiply
the tiles that have already arrived (``csrc/gemm.cu``, ``gemm_ag_launch``). The backward pass
gathers again for ``dx = dy @ W`` (MN-major weight operand, flags per 256 contraction rows) and
forms the full weight gradient locally; the caller (or :class:`AgLinear`) reduce-scatters it.

Reference parity: the reference shards parameters with torch FSDP2 through accelerate
(workspace/lerobot_example/config_qact.yml ``FSDP2: True``; train_qact.py:42-70), i.e. an NCCL
all-gather followed by cuBLAS; this is the fused equivalent. :func:`ag_dual_gate_up` is the same
for the two FFN experts' gate/up projections in one launch
(wall_x/model/qwen2_5_based/modeling_qwen2_5_vl_act.py:228-330, csrc/dual_asym_grouped_gemm.cu:49-136).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..ops import _ext
from ..ops import gemm as G


class GatherWorkspace:
    """Local staging memory shared by all sharded weights of a model (one weight at a time per slot)."""

    def __init__(self, max_elems: int, device, slots: int = 2):
        self.buf = torch.empty(slots, max_elems, dtype=torch.bfloat16, device=device)
        self.max_elems = int(max_elems)

    def view(self, rows: int, cols: int, slot: int = 0) -> torch.Tensor:
        n = rows * cols
        if n > self.max_elems:
            raise ValueError(f"gather workspace holds {self.max_elems} elements, weight needs {n}")
        return self.buf[slot, :n].view(rows, cols)


class ShardedWeight:
    """``rows / world`` rows of a ``[rows, cols]`` bf16 weight in symmetric memory, plus peer addresses."""

    def __init__(self, rows: int, cols: int, group, device, workspace: Optional[GatherWorkspace] = None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if rows % self.world:
            raise ValueError(f"weight rows {rows} must divide evenly over {self.world} ranks")
        if cols % 8:
            raise ValueError("weight row length must be a multiple of 8 elements (16 bytes)")
        self.rows, self.cols = int(rows), int(cols)
        self.rows_per_rank = rows // self.world
        self.group = group
        if torch.device(device).type == "cpu":
            # CPU stand-in (tests of the shard arithmetic over gloo): same row split, the gather is a collective
            self.shard = torch.zeros(self.rows_per_rank, cols, dtype=torch.float32)
            self.peer_ptrs, self.flags, self.epoch, self.workspace = [], None, 0, None
            self.grad = self.full_grad = None
            return
        self.shard = symm_mem.empty(self.rows_per_rank, cols, dtype=torch.bfloat16, device=device)
        self.shard.zero_()
        hdl = symm_mem.rendezvous(self.shard, group)
        self.peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
        self.flags = torch.zeros((rows + 255) // 256, dtype=torch.int32, device=device)
        self.epoch = 0
        self.workspace = workspace if workspace is not None else GatherWorkspace(rows * cols, device, slots=1)
        self.grad: Optional[torch.Tensor] = None  # fp32 [rows_per_rank, cols] after reduce_scatter_grad
        self.full_grad: Optional[torch.Tensor] = None  # fp32 [rows, cols], accumulated by backward passes

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

    def staging(self, slot: int = 0) -> torch.Tensor:
        return self.workspace.view(self.rows, self.cols, slot)

    def next_epoch(self) -> int:
        self.epoch += 1
        if self.epoch >= (1 << 24):  # flags are int32 counts of n_pullers * epoch
            self.flags.zero_()
            self.epoch = 1
        return self.epoch


def ag_launch(specs: Sequence[G.GemmSpec], weights: Sequence[ShardedWeight], n_pullers: int = 0) -> None:
    """One launch of one or two problems; ``specs[i].b`` must be ``weights[i].staging(slot)`` (distinct slots)."""
    _ext.get().gemm_ag([s.as_tuple() for s in specs], [w.peer_ptrs for w in weights], [w.flags for w in weights],
                       weights[0].rank, [w.rows_per_rank for w in weights], int(n_pullers),
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


class _AgLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, anchor, w: ShardedWeight, bias, n_pullers):
        ctx.w, ctx.n_pullers, ctx.has_bias = w, n_pullers, bias is not None
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2)
        y = ag_gemm(x2, w, bias=bias, n_pullers=n_pullers)
        return y.view(*x.shape[:-1], w.rows)

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        w = ctx.w
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = ag_gemm(dy2, w, transpose_w=True, n_pullers=ctx.n_pullers)
        # full weight gradient, fp32, accumulated over micro-batches; reduce-scattered by the owner
        if w.full_grad is None:
            w.full_grad = torch.zeros(w.rows, w.cols, dtype=torch.float32, device=dy.device)
        if dy2.is_cuda:
            G.launch([G.GemmSpec(dy2, x2, w.full_grad, a_mn=True, b_mn=True, flags=G.OUT_FP32 | G.ACCUMULATE)])
        else:
            w.full_grad += dy2.float().t() @ x2.float()
        dbias = dy2.float().sum(0).to(dy.dtype) if ctx.has_bias else None
        return dx.view(*dy.shape[:-1], w.cols), None, None, dbias, None


class AgLinear(torch.nn.Module):
    """``nn.Linear`` whose weight lives as a :class:`ShardedWeight`; the gather is fused into the GEMMs."""

    def __init__(self, in_features: int, out_features: int, group, device, bias: bool = False,
                 workspace: Optional[GatherWorkspace] = None, n_pullers: int = 0):
        super().__init__()
        self.weight = ShardedWeight(out_features, in_features, group, device, workspace)
        self.group = group
        self.n_pullers = n_pullers
        bdt = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
        self.bias = torch.nn.Parameter(torch.zeros(out_features, dtype=bdt, device=device)) if bias else None
        # autograd needs one differentiable input even when x does not require grad
        self._anchor = torch.nn.Parameter(torch.zeros((), device=device))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _AgLinearFn.apply(x, self._anchor, self.weight, self.bias, self.n_pullers)

    def reduce_scatter_grad(self) -> torch.Tensor:
        """Average the full fp32 gradients over ranks and keep this rank's rows (``weight.grad``)."""
        import torch.distributed as dist

        w = self.weight
        out = torch.empty(w.rows_per_rank, w.cols, dtype=torch.float32, device=w.shard.device)
        if w.full_grad.is_cuda:
            dist.reduce_scatter_tensor(out, w.full_grad, op=dist.ReduceOp.AVG, group=self.group)
        else:  # gloo has no reduce-scatter: all-reduce and keep this rank's rows
            dist.all_reduce(w.full_grad, op=dist.ReduceOp.SUM, group=self.group)
            r0 = w.rank * w.rows_per_rank
            out.copy_(w.full_grad[r0:r0 + w.rows_per_rank] / w.world)
        w.full_grad = None
        w.grad = out
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

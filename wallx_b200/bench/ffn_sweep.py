"""Kernel sweep of the dual-expert FFN path: permute -> two-expert gate/up/down GEMMs -> unpermute.

``python -m wallx_b200.bench.ffn_sweep [--impl ours|reference] [--tokens 2048,8192,32768]
[--fracs 0.05,0.25,0.5] [--out FILE]`` at hidden 2048, bf16, VLM expert width 11008, action expert
width from the model config; action tokens sit at random positions. One JSON line per case with
device-timed forward and forward+backward times and the achieved fraction of the measured GEMM
peak.

Launched under ``torch.distributed.run`` with N > 1 ranks, the expert weights are sharded by rows
over the ranks and the forward is timed with the weight all-gather fused into the GEMMs
(``parallel/ag_linear.py``); the roofline is then the slower of FLOPs / GEMM peak and gathered
bytes / NVLink bandwidth. ``--impl reference`` runs the installed reference's own
``SparseMoeBlock`` (its permute / unpermute CUDA ops around per-expert cuBLAS Linears,
wall_x/model/qwen2_5_based/modeling_qwen2_5_vl_act.py:85-160), wrapped in torch FSDP2
``fully_shard`` for N > 1 (NCCL all-gather, then cuBLAS).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

HIDDEN = 2048
VLM_FFN = 11008
NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), "of measured"
    except Exception:
        return 1590.0, "of fallback"


def _time(fn, iters, warmup, barrier):
    for _ in range(warmup):
        fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    barrier()
    return e0.elapsed_time(e1) / iters


def _types(T, frac, seed):
    g = torch.Generator().manual_seed(seed)
    n_act = int(round(T * frac))
    tt = torch.zeros(T, dtype=torch.int64)
    tt[torch.randperm(T, generator=g)[:n_act]] = 1
    return tt, n_act


def run_ours(args, dev, world, rank, barrier):
    from wallx_b200.ops import _ext
    from wallx_b200.ops import functional as F_
    from wallx_b200.ops import gemm as G
    from wallx_b200.models.layers import SwiGLUFFN

    C = _ext.get()
    widths = (VLM_FFN, args.action_ffn)
    torch.manual_seed(0)
    experts = [SwiGLUFFN(HIDDEN, w, bias=False).to(torch.bfloat16).to(dev) for w in widths]
    for e in experts:
        for p in e.parameters():
            torch.nn.init.normal_(p, std=0.02)
    weights = [e.weights() for e in experts]
    sharded = None
    if world > 1:
        import torch.distributed as dist

        from wallx_b200.parallel.ag_linear import GatherWorkspace, ShardedWeight, ag_launch

        ws = GatherWorkspace(2 * VLM_FFN * HIDDEN, dev, slots=2)
        sharded = []
        for wgu, wdn in weights:
            pair = []
            for w in (wgu, wdn):
                sw = ShardedWeight(w.shape[0], w.shape[1], dist.group.WORLD, dev, ws)
                sw.load_full(w.detach())
                pair.append(sw)
            sharded.append(pair)
        torch.cuda.synchronize()
        dist.barrier()
        zero3 = None
        if not args.no_bwd:
            # the training-engine form of the same four weights: one row-sharded unit in symmetric memory
            from wallx_b200.parallel.symm import SymmComm
            from wallx_b200.parallel.zero3 import GatherWorkspace as GW, RowShardedBuffer

            symm = SymmComm(dist.group.WORLD, dev)
            named = []
            for e, ex in enumerate(experts):
                twin = SwiGLUFFN(HIDDEN, widths[e], bias=False).to(torch.bfloat16).to(dev)
                twin.load_state_dict(ex.state_dict())
                named += [(f"moe.experts.{e}.gate_up_weight", twin.gate_up_weight), (f"moe.experts.{e}.down_weight", twin.down_weight)]
            a, b = RowShardedBuffer.sizes([p for _, p in named], world)
            symm.reserve(a, dtype=torch.bfloat16, grad_elems=b)
            buf = RowShardedBuffer(named, world, rank, name="ffn", alloc=(symm.alloc_param, symm.alloc_grad), mode="gathered")
            symm.register_buffers([buf])
            ws2 = GW(max(R * C for R, C in buf.shapes), dev, slots=2)
            flags = torch.zeros(buf.flag_words(), dtype=torch.int32, device=dev)
            buf.attach_gather(symm.param_ptrs, ws2, flags)
            zero3 = {"symm": symm, "buf": buf, "weights": [(named[0][1], named[1][1]), (named[2][1], named[3][1])]}
            torch.cuda.synchronize()
            dist.barrier()
    out = []
    for T in args.tokens:
        for frac in args.fracs:
            tt, n_act = _types(T, frac, 17)
            xs = [torch.randn(T, HIDDEN, device=dev).to(torch.bfloat16).requires_grad_(True) for _ in range(2)]
            plan = F_.make_route_plan(tt.to(dev), 2)
            dy = torch.randn(T, HIDDEN, device=dev).to(torch.bfloat16)
            it = [0]

            def fwd_local():
                x = xs[it[0] & 1]
                it[0] += 1
                xp = C.permute_rows(x.detach(), plan.dest, plan.rows)
                return F_.moe_ffn(xp, None, plan, weights)

            def fwd_bwd_local():
                x = xs[it[0] & 1]
                it[0] += 1
                xp = _PermuteFn.apply(x, plan)
                y = F_.moe_ffn(xp, None, plan, weights)
                y.backward(dy)
                x.grad = None
                for wgu, wdn in weights:
                    wgu.grad = None
                    wdn.grad = None

            def fwd_sharded():
                x = xs[it[0] & 1]
                it[0] += 1
                xp = C.permute_rows(x.detach(), plan.dest, plan.rows)
                rows = plan.rows
                h = torch.empty(rows, VLM_FFN, device=dev, dtype=torch.bfloat16)
                y = torch.empty(T, HIDDEN, device=dev, dtype=torch.bfloat16)
                sp = [G.GemmSpec(xp, sharded[e][0].staging(e), h, M=rows, dyn=plan.seg[e],
                                 flags=G.ACT_SWIGLU | G.ZERO_PAD_ROWS) for e in range(2)]
                ag_launch(sp, [sharded[e][0] for e in range(2)])
                sp = [G.GemmSpec(h[:, :widths[e]], sharded[e][1].staging(e), y, M=rows, dyn=plan.seg[e], row_map=plan.inv)
                      for e in range(2)]
                ag_launch(sp, [sharded[e][1] for e in range(2)])
                return y

            def fwd_bwd_sharded():
                # what one layer's FFN costs in a ZeRO-3 training step: forward and dgrad GEMMs gather the weights from
                # their owners inside the kernels, the wgrad GEMMs add into local bf16 buffers, and every rank reduces its
                # rows of those buffers by peer loads (csrc/comm.cu rs_reduce) behind a flag barrier
                x = xs[it[0] & 1]
                it[0] += 1
                xp = _PermuteFn.apply(x, plan)
                y = F_.moe_ffn(xp, None, plan, zero3["weights"])
                y.backward(dy)
                x.grad = None
                zero3["symm"].begin_step()
                zero3["symm"].reduce_scatter_unit(0)
                zero3["buf"].grad.zero_()

            flops_f = 2.0 * HIDDEN * 3 * ((T - n_act) * widths[0] + n_act * widths[1])
            rec = {"impl": "ours", "tokens": T, "action_frac": frac, "n_gpus": world, "hidden": HIDDEN,
                   "ffn": list(widths), "dtype": "bf16"}
            with torch.no_grad():
                if sharded is None:
                    rec["fwd_ms"] = _time(fwd_local, args.iters, args.warmup, barrier)
                else:
                    rec["fwd_ms"] = _time(fwd_sharded, args.iters, args.warmup, barrier)
                    rec["path"] = "weight all-gather fused into the GEMMs (peer loads, no NCCL)"
                    rec["fwd_local_ms"] = _time(fwd_local, args.iters, args.warmup, barrier)
                    # parity of the two forwards
                    it[0] = 0
                    a = fwd_sharded()
                    it[0] = 0
                    b = fwd_local()
                    rec["max_abs_diff_vs_unsharded"] = float((a.float() - b.float()).abs().max())
            if sharded is None and not args.no_bwd:
                rec["fwd_bwd_ms"] = _time(fwd_bwd_local, args.iters, args.warmup, barrier)
            if sharded is not None and not args.no_bwd:
                rec["fwd_bwd_ms"] = _time(fwd_bwd_sharded, args.iters, args.warmup, barrier)
                rec["fwd_bwd_path"] = "gathers fused into forward + dgrad GEMMs, bf16 wgrad, peer-load reduce-scatter of the owner's rows"
                zero3["symm"].check()
            G.check_status()
            out.append((rec, flops_f))
    return out


class _PermuteFn(torch.autograd.Function):
    """Row gather into expert order and its adjoint (used only to time a standalone permute)."""

    @staticmethod
    def forward(ctx, x, plan):
        from wallx_b200.ops import _ext

        ctx.plan = plan
        return _ext.get().permute_rows(x, plan.dest, plan.rows)

    @staticmethod
    def backward(ctx, g):
        from wallx_b200.ops import _ext

        return _ext.get().gather_rows(g.contiguous(), ctx.plan.dest), None


def run_reference(args, dev, world, rank, barrier):
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ref_dir = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "wall_x")):
        return "baseline/_ref/wall_x is not installed on this box"
    from . import ref_shims

    ref_shims.install(ref_dir)
    from wall_x.model.qwen2_5_based.modeling_qwen2_5_vl_act import SparseMoeBlock  # reference

    class _Cfg:
        experts = [{"hidden_size": HIDDEN, "intermediate_size": VLM_FFN, "hidden_act": "silu"},
                   {"hidden_size": HIDDEN, "intermediate_size": args.action_ffn, "hidden_act": "silu"}]

    torch.manual_seed(0)
    blk = SparseMoeBlock(_Cfg(), 2).to(torch.bfloat16).to(dev)
    for p in blk.parameters():
        torch.nn.init.normal_(p, std=0.02)
    if args.ref_path == "cutlass":
        # The reference ships a CUTLASS grouped GEMM for the two experts (csrc/dual_asym_grouped_gemm.cu:308-366,
        # wrapper wall_x/fusions/ops.py:147) that its model never calls. This is that kernel put where the expert loop
        # is: the reference's own permute / unpermute ops around three asym_dual_gmm launches and an unfused SiLU * up.
        from wall_x.fusions import ops as ref_ops  # reference

        class CutlassMoe(torch.nn.Module):
            def __init__(self, inner):
                super().__init__()
                self.experts = inner.experts

            def forward(self, hidden_states, experts_indices, start, end):
                b, s_, h = hidden_states.size()
                x = hidden_states.view(-1, h)
                idx = experts_indices.view(-1)
                probs = torch.ones_like(idx, dtype=torch.float32).view(-1, 1)
                xp, row_map = ref_ops.permute(x, idx)
                e0, e1 = self.experts[0], self.experts[1]
                x0, x1 = xp[start[0]:end[0]], xp[start[1]:end[1]]
                g0, g1 = ref_ops.asym_dual_gmm(x0, x1, e0.gate_proj.weight, e1.gate_proj.weight, trans_b=True)
                u0, u1 = ref_ops.asym_dual_gmm(x0, x1, e0.up_proj.weight, e1.up_proj.weight, trans_b=True)
                h0, h1 = torch.nn.functional.silu(g0) * u0, torch.nn.functional.silu(g1) * u1
                y0, y1 = ref_ops.asym_dual_gmm(h0, h1, e0.down_proj.weight, e1.down_proj.weight, trans_b=True)
                return ref_ops.unpermute(torch.cat([y0, y1], dim=0), row_map, probs).view(b, s_, h)

        blk = CutlassMoe(blk)
    if world > 1:
        from torch.distributed.fsdp import fully_shard

        fully_shard(blk, reshard_after_forward=True)
    out = []
    for T in args.tokens:
        for frac in args.fracs:
            tt, n_act = _types(T, frac, 17)
            ttd = tt.to(dev).view(1, T)
            sizes = torch.tensor([T - n_act, n_act])
            start, end = torch.cumsum(sizes, 0) - sizes, torch.cumsum(sizes, 0)
            xs = [torch.randn(1, T, HIDDEN, device=dev).to(torch.bfloat16).requires_grad_(True) for _ in range(2)]
            dy = torch.randn(1, T, HIDDEN, device=dev).to(torch.bfloat16)
            it = [0]

            def fwd():
                x = xs[it[0] & 1]
                it[0] += 1
                return blk(x.detach(), ttd, start, end)

            def fwd_bwd():
                x = xs[it[0] & 1]
                it[0] += 1
                blk(x, ttd, start, end).backward(dy)
                x.grad = None
                blk.zero_grad(set_to_none=True)

            flops_f = 2.0 * HIDDEN * 3 * ((T - n_act) * VLM_FFN + n_act * args.action_ffn)
            rec = {"impl": "reference", "ref_path": args.ref_path, "tokens": T, "action_frac": frac, "n_gpus": world,
                   "hidden": HIDDEN, "ffn": [VLM_FFN, args.action_ffn], "dtype": "bf16"}
            with torch.no_grad():
                rec["fwd_ms"] = _time(fwd, args.iters, args.warmup, barrier)
            if world > 1:
                rec["path"] = ("torch FSDP2 fully_shard (NCCL all-gather, reduce-scatter in backward) + reference permute/unpermute + "
                               + ("cuBLAS" if args.ref_path == "cublas" else "CUTLASS asym_dual_gmm"))
            if not args.no_bwd:
                rec["fwd_bwd_ms"] = _time(fwd_bwd, args.iters, args.warmup, barrier)
            out.append((rec, flops_f))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", default="2048,8192,32768")
    ap.add_argument("--fracs", default="0.05,0.25,0.5")
    ap.add_argument("--action-ffn", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--no-bwd", action="store_true")
    ap.add_argument("--ref-path", default="cublas", choices=["cublas", "cutlass"],
                    help="reference arm: its shipped model path (per-expert cuBLAS loop) or its dormant CUTLASS grouped GEMM")
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    args.tokens = [int(t) for t in args.tokens.split(",")]
    args.fracs = [float(f) for f in args.fracs.split(",")]
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    res = run_ours(args, dev, world, rank, barrier) if args.impl == "ours" else run_reference(args, dev, world, rank, barrier)
    if isinstance(res, str):
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": res}))
        return
    peak, tag = _peaks()
    lines = []
    for rec, flops_f in res:
        # max over ranks of every timing
        keys = [k for k in ("fwd_ms", "fwd_local_ms", "fwd_bwd_ms") if k in rec]
        t = torch.tensor([rec[k] for k in keys], device=dev, dtype=torch.float64)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        for k, v in zip(keys, t.tolist()):
            rec[k] = round(v, 4)
        rec["fwd_tflops"] = round(flops_f / rec["fwd_ms"] / 1e9, 1)
        t_compute = flops_f / (peak * 1e12) * 1e3
        t_link = 0.0
        if world > 1:
            wbytes = 3 * HIDDEN * (VLM_FFN + args.action_ffn) * 2
            t_link = wbytes * (world - 1) / world / (NVLINK_GBS * 1e9) * 1e3
            rec["roofline"] = {"compute_ms": round(t_compute, 4), "nvlink_ms": round(t_link, 4)}
        rec["fwd_frac_of_roofline"] = round(max(t_compute, t_link) / rec["fwd_ms"], 3)
        rec["roofline_basis"] = f"{peak} TFLOP/s cuBLAS bf16 burst {tag}" + (f", {NVLINK_GBS} GB/s NVLink" if world > 1 else "")
        if "fwd_bwd_ms" in rec:
            rec["fwd_bwd_tflops"] = round(3 * flops_f / rec["fwd_bwd_ms"] / 1e9, 1)
        lines.append(json.dumps(rec))
    if rank == 0:
        for ln in lines:
            print(ln, flush=True)
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            with open(args.out, "a") as f:
                f.write("\n".join(lines) + "\n")
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())

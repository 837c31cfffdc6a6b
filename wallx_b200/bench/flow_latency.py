"""Flow-matching inference latency at WALL-OSS-FLOW size: p50 / p99 per action chunk.

``python -m wallx_b200.bench.flow_latency [--impl ours|reference] [--batch 1,32] [--chunks 30]``

One chunk = the host-to-device copy of one observation (3 views of 256x256, 64 prompt tokens,
20-d proprioception) from pinned memory, the ViT + prefix pass that fills the KV cache, 10 Euler
evaluations of the velocity field over a 32x20 action chunk drawn from N(0, 1) reusing the prefix
KV, un-normalisation, and the device-to-host read of the predicted chunk. Every chunk is timed with
its own CUDA event pair on the launching stream. Under ``torch.distributed.run`` with N ranks the
model is replicated and each rank serves its own stream of chunks; the reported percentile is the
max over ranks.

``--impl reference`` runs the installed reference's own ``model(mode="predict",
predict_mode="diffusion")`` (modeling_qwen2_5_vl_act.py:1886-1981: every evaluation re-runs the whole
sequence) with ``num_inference_timesteps=11``, which is 10 evaluations on its ``linspace`` grid.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _percentile(xs, q):
    xs = sorted(xs)
    k = (len(xs) - 1) * q
    lo = int(k)
    hi = min(lo + 1, len(xs) - 1)
    return xs[lo] + (xs[hi] - xs[lo]) * (k - lo)


def _pin(b):
    return {k: (v.pin_memory() if isinstance(v, torch.Tensor) else v) for k, v in b.items()}


def _h2d(b, dev, float_dtype):
    out, nbytes = {}, 0
    for k, v in b.items():
        if isinstance(v, torch.Tensor):
            nbytes += v.numel() * v.element_size()
            v = v.to(dev, non_blocking=True)
            if v.is_floating_point():
                v = v.to(float_dtype)
        out[k] = v
    return out, nbytes


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", default="1,32")
    ap.add_argument("--chunks", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--steps", type=int, default=10, help="Euler evaluations per chunk")
    ap.add_argument("--action-ffn", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer decoder layers")
    ap.add_argument("--cuda-graph", action="store_true", help="ours: capture the Euler loop in a CUDA graph")
    ap.add_argument("--engine", action="store_true",
                    help="ours: FlowEngine (fixed observation layout, static buffers, one CUDA graph per chunk)")
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)

    from wallx_b200.config import wall_oss_config
    from wallx_b200.data.synthetic import make_batch, make_processor

    cfg = wall_oss_config(action_expert_intermediate=args.action_ffn,
                          **({"num_hidden_layers": args.layers} if args.layers else {}))
    proc = make_processor(cfg, 2048)
    torch.manual_seed(1234)
    if args.impl == "ours":
        from wallx_b200.models import Qwen2_5_VLMoEForAction

        model = Qwen2_5_VLMoEForAction(cfg, processor=proc).to(torch.bfloat16).to(dev)
        model.init_weights(seed=0)
    else:
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        ref_dir = os.path.join(root, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "wall_x")):
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/wall_x is not installed on this box"}))
            return
        from . import ref_shims
        from .reference_arm import _build_model

        ref_shims.install(ref_dir)

        class _A:
            action_ffn, layers, mode = args.action_ffn, args.layers, "flow"

        _, proc, model = _build_model(_A, dev)
    model.eval()

    lines = []
    for B in [int(b) for b in args.batch.split(",")]:
        gen = torch.Generator().manual_seed(100 + rank)
        pool = []
        for _ in range(3):
            b = make_batch(cfg, proc, B, views=3, image_hw=(256, 256), prompt_len=64, horizon=32, mode="flow", generator=gen)
            b.pop("action_chunk", None)
            b.pop("labels", None)
            pool.append(_pin(b))
        seq_len = int(pool[0]["input_ids"].shape[1])

        engine = None
        if args.engine and args.impl == "ours":
            from wallx_b200.models.inference import FlowEngine

            engine = FlowEngine(model, pool[0], num_inference_timesteps=args.steps)

        def chunk(i):
            if engine is not None:
                host_batch = pool[i % len(pool)]
                nbytes = sum(host_batch[k].numel() * host_batch[k].element_size() for k in engine.static if k in host_batch)
                out = engine(host_batch)  # H2D straight into the static buffers, graph replay
                return nbytes, out["predict_action"].float().cpu()
            batch, nbytes = _h2d(pool[i % len(pool)], dev, torch.bfloat16)
            with torch.no_grad():
                if args.impl == "ours":
                    out = model(mode="predict", predict_mode="diffusion", num_inference_timesteps=args.steps,
                                use_cuda_graph=args.cuda_graph, **batch)
                else:
                    out = model(mode="predict", predict_mode="diffusion", num_inference_timesteps=args.steps + 1,
                                pred_horizon=32, action_dim=20, **batch)
            host = out["predict_action"].float().cpu()
            return nbytes, host

        for i in range(args.warmup):
            chunk(i)
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
        times = []
        for i in range(args.chunks):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            nbytes, host = chunk(i)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        p = torch.tensor([_percentile(times, 0.5), _percentile(times, 0.99), sum(times) / len(times)], device=dev,
                         dtype=torch.float64)
        if world > 1:
            torch.distributed.all_reduce(p, op=torch.distributed.ReduceOp.MAX)
        rec = {"metric": "flow action-chunk latency (ms), H2D of the observation to D2H of the chunk",
               "impl": args.impl, "batch": B, "n_gpus": world, "p50_ms": round(float(p[0]), 3),
               "p99_ms": round(float(p[1]), 3), "mean_ms": round(float(p[2]), 3), "chunks": args.chunks,
               "euler_evaluations": args.steps, "seq_len": seq_len, "dtype": "bf16", "data": "synthetic",
               "h2d_bytes_per_chunk": int(nbytes), "d2h_bytes_per_chunk": int(host.numel() * 4),
               "chunks_per_s_total": round(world * B * 1e3 / float(p[2]), 2),
               "config": ("WALL-OSS-FLOW size, 36 layers, 3x256x256 views, 64 prompt tokens, 32x20 chunk"
                          + (f" DEBUG layers={args.layers}" if args.layers else "")
                          + (", CUDA-graph Euler loop" if args.cuda_graph and args.impl == "ours" else "")
                          + (", FlowEngine: whole chunk in one CUDA graph" if engine is not None else ""))}
        lines.append(json.dumps(rec))
        if rank == 0:
            print(lines[-1], flush=True)
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "a") as f:
            f.write("\n".join(lines) + "\n")
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())

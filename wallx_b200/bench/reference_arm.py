"""Reference arm of the benchmark.

Runs the unmodified reference package installed under ``baseline/_ref`` (its own model classes,
its own CUDA extension ``wallx_csrc``, flash-attn 2, cuBLAS, NCCL) for the same metric and
configuration as ``bench.py``'s own arm and prints the same JSON line with ``"impl": "reference"``.

The reference's trainer is a thin loop over ``accelerate`` (not on this image), so the loop here
restates it with the same calls in the same order (train_qact.py:42-70 and
qwen_vl_act_trainer.py:313-343): ``model(**batch, mode="train")`` -> ``loss / accum`` backward ->
``clip_grad_norm_(1.0)`` -> ``AdamW.step`` on bf16 parameters (bf16 Adam states, as the reference
casts the model before building the optimizer, :527,577-581) -> ``zero_grad``; for N > 1 the model
is wrapped with torch FSDP2 ``fully_shard`` per decoder layer / vision block with
``reshard_after_forward=True``, which is what accelerate's FSDP2 plugin sets up. None of this
framework's models, kernels or engine is on that path; only the synthetic batch generator (plain
tensors) is shared so that both arms see the same data.
"""
from __future__ import annotations

import json
import os
import sys


def unavailable(reason: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": reason}), flush=True)


def _build_model(args, dev):
    import torch

    from wall_x.model.qwen2_5_based.configuration_qwen2_5_vl import Qwen2_5_VLConfig  # reference
    from wall_x.model.qwen2_5_based.modeling_qwen2_5_vl_act import Qwen2_5_VLMoEForAction  # reference

    from wallx_b200.config import wall_oss_config
    from wallx_b200.data.synthetic import make_processor

    ours = wall_oss_config(action_expert_intermediate=args.action_ffn,
                           **({"num_hidden_layers": args.layers} if args.layers else {}))
    d = ours.to_dict()
    for k in ("architectures", "model_type", "mrope_layout", "action_attn", "output_attentions", "output_hidden_states",
              "use_return_dict"):
        d.pop(k, None)
    d["vision_config"]["initializer_range"] = 0.02
    cfg = Qwen2_5_VLConfig(**d)
    cfg._attn_implementation = "flash_attention_2"
    cfg.vision_config._attn_implementation = "flash_attention_2"
    proc = make_processor(ours, 2048)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = Qwen2_5_VLMoEForAction(cfg, use_fast_tokenizer=(args.mode == "fast"), processor=proc)
    finally:
        torch.set_default_dtype(old)
    model = model.to(torch.bfloat16)
    return ours, proc, model


def _train_arm(args, mode, world, rank, local, dev, steps, warmup, do_e2e):
    """Build the reference model for ``mode`` and time ``steps`` training steps. Returns a dict of raw numbers."""
    import torch
    import torch.distributed as dist

    from wallx_b200.data.synthetic import make_batch

    class _A:
        pass

    a = _A()
    a.action_ffn, a.layers, a.mode = args.action_ffn, args.layers, mode
    torch.manual_seed(1234)
    ours_cfg, proc, model = _build_model(a, dev)
    model.train()
    accum = max(1, args.per_gpu_batch // args.micro_batch)
    micro = args.per_gpu_batch // accum
    if world > 1:
        from torch.distributed.fsdp import fully_shard

        for blk in model.visual.blocks:
            fully_shard(blk, reshard_after_forward=True)
        for layer in model.model.layers:
            fully_shard(layer, reshard_after_forward=True)
        fully_shard(model, reshard_after_forward=True)
    params = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, lr=9e-5, weight_decay=0.1)

    gen = torch.Generator().manual_seed(100 + rank)
    pool = []
    for _ in range(2):
        mbs = []
        for _a in range(accum):
            b = make_batch(ours_cfg, proc, micro, views=3, image_hw=(256, 256), prompt_len=64, horizon=32, mode=mode,
                           fast_tokens=48, generator=gen)
            b = {k: (v.pin_memory() if isinstance(v, torch.Tensor) else v) for k, v in b.items()}
            mbs.append(b)
        pool.append(mbs)

    def stage(b):
        out = {}
        for k, v in b.items():
            if isinstance(v, torch.Tensor):
                v = v.to(dev, non_blocking=True)
                if v.is_floating_point():
                    v = v.to(torch.bfloat16)
            out[k] = v
        return out

    def h2d_bytes(b):
        return sum(v.numel() * v.element_size() for v in b.values() if isinstance(v, torch.Tensor))

    def train_step(mbs):
        loss = None
        for mb in mbs:
            out = model(**mb, mode="train")
            (out.loss / accum).backward()
            loss = out.loss.detach()
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        opt.step()
        opt.zero_grad()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    resident = [[stage(b) for b in mbs] for mbs in pool]
    for i in range(warmup):
        train_step(resident[i % len(resident)])
    barrier()

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    from bench import ClockSampler

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(steps):
        loss = train_step(resident[i % len(resident)])
    e1.record()
    barrier()
    ms_dev = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    loss_val = float(loss.item())

    ms_e2e = 0.0
    bi = 0
    if do_e2e:
        train_step([stage(b) for b in pool[0]])
        barrier()
        e0.record()
        for i in range(steps):
            l = train_step([stage(b) for b in pool[i % len(pool)]])
            _ = l.float().cpu()
        e1.record()
        barrier()
        ms_e2e = e0.elapsed_time(e1)
        bi = sum(h2d_bytes(b) for b in pool[0])
    t = torch.tensor([ms_dev, ms_e2e, torch.cuda.max_memory_allocated(dev) / 2 ** 30], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res = {"ms_dev": float(t[0]), "ms_e2e": float(t[1]), "peak_gb": float(t[2]), "clocks": clocks, "loss": loss_val,
           "h2d": int(bi), "accum": accum, "micro": micro, "seq_len": int(pool[0][0]["input_ids"].shape[1])}
    del model, opt, params, resident, pool
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    return res


def _latency_block(args, world, rank, dev, chunks):
    """p50 / p99 of the reference's own ``model(mode="predict", predict_mode="diffusion")`` per action chunk, H2D of
    the observation to D2H of the chunk, with ``num_inference_timesteps=11`` (10 evaluations on its linspace grid;
    every evaluation re-runs the whole sequence, modeling_qwen2_5_vl_act.py:1906-1962)."""
    import torch
    import torch.distributed as dist

    from wallx_b200.bench.flow_latency import _h2d, _percentile, _pin
    from wallx_b200.data.synthetic import make_batch

    class _A:
        pass

    a = _A()
    a.action_ffn, a.layers, a.mode = args.action_ffn, args.layers, "flow"
    torch.manual_seed(1234)
    ours_cfg, proc, model = _build_model(a, dev)
    model.eval()
    out = {"unit": "ms per chunk", "euler_evaluations": 10, "chunks": chunks,
           "path": "reference predict(diffusion), num_inference_timesteps=11; timed H2D of the observation to D2H of the chunk"}
    for B in (1, 32):
        gen = torch.Generator().manual_seed(100 + rank)
        pool = []
        for _ in range(3):
            b = make_batch(ours_cfg, proc, B, views=3, image_hw=(256, 256), prompt_len=64, horizon=32, mode="flow", generator=gen)
            b.pop("action_chunk", None)
            b.pop("labels", None)
            pool.append(_pin(b))

        def chunk(i):
            batch, _ = _h2d(pool[i % 3], dev, torch.bfloat16)
            with torch.no_grad():
                o = model(mode="predict", predict_mode="diffusion", num_inference_timesteps=11, pred_horizon=32,
                          action_dim=20, **batch)
            return o["predict_action"].float().cpu()

        for i in range(2):
            chunk(i)
        torch.cuda.synchronize()
        times = []
        for i in range(chunks):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            chunk(i)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        p = torch.tensor([_percentile(times, 0.5), _percentile(times, 0.99)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(p, op=dist.ReduceOp.MAX)
        out[f"batch{B}"] = {"p50_ms": round(float(p[0]), 3), "p99_ms": round(float(p[1]), 3)}
    return out


def main(args) -> None:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ref_dir = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "wall_x")):
        return unavailable("baseline/_ref/wall_x is not installed on this box")
    import torch

    if not torch.cuda.is_available():
        return unavailable("no CUDA device (the reference's action head and fused ops are CUDA-only)")
    import torch.distributed as dist

    from . import ref_shims

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    try:
        ref_shims.install(ref_dir)
        if world > 1:
            dist.init_process_group("nccl", device_id=dev)
    except Exception as e:  # the reference could not be brought up on this software stack
        import traceback

        traceback.print_exc(file=sys.stderr)
        return unavailable(f"reference could not be constructed: {type(e).__name__}: {str(e)[:200]}")
    try:
        r = _train_arm(args, args.mode, world, rank, local, dev, args.steps, args.warmup, not args.no_e2e)
    except Exception as e:
        import traceback

        traceback.print_exc(file=sys.stderr)
        return unavailable(f"reference training step failed: {type(e).__name__}: {str(e)[:200]}")
    gb = args.per_gpu_batch * world
    rec = {
        "metric": f"train samples/s, WALL-OSS-{args.mode.upper()}-size fine-tune (max over ranks, device-timed)",
        "value": round(gb * args.steps / (r["ms_dev"] / 1e3), 3), "unit": "samples/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(r["ms_dev"] / args.steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"model": f"WALL-OSS-{args.mode.upper()} (reference classes, flash_attention_2, action expert FFN {args.action_ffn})"
                            + (f" DEBUG layers={args.layers}" if args.layers else ""),
                   "global_batch": gb, "per_gpu_batch": args.per_gpu_batch, "micro_batch": r["micro"], "grad_accum": r["accum"],
                   "seq_len": r["seq_len"],
                   "parallelism": ("fsdp2 fully_shard per layer/block, reshard_after_forward, NCCL" if world > 1 else "single GPU"),
                   "optimizer": "torch.optim.AdamW on bf16 params (bf16 states), clip 1.0", "loss": r["loss"],
                   "peak_device_memory_gb": round(r["peak_gb"], 1)},
        "clocks": r["clocks"],
    }
    if not args.no_e2e:
        rec["e2e"] = {"value": round(gb * args.steps / (r["ms_e2e"] / 1e3), 3), "unit": "samples/s",
                      "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": 4, "ms_per_step": round(r["ms_e2e"] / args.steps, 3)}

    def extra(name, fn):
        try:
            rec[name] = fn()
        except Exception as e:
            import traceback

            traceback.print_exc(file=sys.stderr)
            rec[name] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
        if world > 1:
            dist.barrier()

    def fast_block():
        torch.cuda.reset_peak_memory_stats(dev)
        k = max(2, min(args.steps, getattr(args, "extra_steps", 4)))
        f = _train_arm(args, "fast", world, rank, local, dev, k, 2, False)
        return {"value": round(gb * k / (f["ms_dev"] / 1e3), 3), "unit": "samples/s", "ms_per_step": round(f["ms_dev"] / k, 3),
                "steps": k, "warmup": 2, "n_gpus": world, "peak_device_memory_gb": round(f["peak_gb"], 1), "loss": f["loss"]}

    if not getattr(args, "no_extras", False):
        if args.mode == "flow":
            extra("fast", fast_block)
        extra("latency", lambda: _latency_block(args, world, rank, dev, max(5, getattr(args, "latency_chunks", 20) // 2)))
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.destroy_process_group()

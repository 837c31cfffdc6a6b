"""Headline benchmark: FSDP-style fine-tune throughput (samples/s) of the WALL-OSS-size VLA model.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference] [--mode flow|fast]

One "step" is one optimizer step over the global batch (per-GPU batch 32 = micro-batch x
accumulation; global batch 32 x N, i.e. 256 on 8 GPUs: weak scaling). Inputs are synthetic
(uniform uint8 camera frames, uniform prompt ids, N(0,1) proprio, uniform actions) and the weights
are random-init at the named architecture. Rank 0 prints one JSON line.

``value`` is timed on the device (CUDA events, barrier + synchronize on both sides, max over
ranks) with inputs already resident; ``e2e`` repeats the measurement through the public training
call with, every step, the host-to-device copy of that step's inputs from pinned memory and a
device-to-host read of the loss.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="flow", choices=["flow", "fast"])
    ap.add_argument("--per-gpu-batch", type=int, default=32)
    ap.add_argument("--micro-batch", type=int, default=32)
    ap.add_argument("--action-ffn", type=int, default=2048, help="action expert FFN width (not in the reference repo)")
    ap.add_argument("--transport", default="auto", choices=["auto", "dist", "symm"])
    ap.add_argument("--layers", type=int, default=0, help="debug only: override depth (invalidates the number)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-overlap-reduce", action="store_true",
                    help="N > 1, own transport: reduce-scatter after backward instead of per unit during it")
    ap.add_argument("--shard-params", action="store_true",
                    help="headline arm with ZeRO-3 row-sharded layer weights (default: resident bf16 parameters)")
    ap.add_argument("--no-extras", action="store_true", help="skip the zero3 / fast / latency blocks after the headline")
    ap.add_argument("--extra-steps", type=int, default=4, help="timed steps of each extra training block")
    ap.add_argument("--latency-chunks", type=int, default=20)
    ap.add_argument("--kernel-table", default="", help="after the timed runs, trace one more step and write per-kernel time shares here")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx = float(parts[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def run_reference(args):
    from wallx_b200.bench import reference_arm

    reference_arm.main(args)


class Arm:
    """One model + engine + synthetic data pool of the training benchmark (one parameter plan, one loss mode)."""

    def __init__(self, args, mode: str, shard: bool, world: int, rank: int, dev, symm_factory):
        import torch

        from wallx_b200.config import wall_oss_config
        from wallx_b200.data.collator import add_pack_info, pin_batch, to_device
        from wallx_b200.data.synthetic import images_to_patches, make_batch, make_processor
        from wallx_b200.models import Qwen2_5_VLMoEForAction
        from wallx_b200.parallel.engine import TrainEngine

        self.args, self.mode, self.shard, self.world, self.rank, self.dev = args, mode, shard, world, rank, dev
        cfg_kw = {"num_hidden_layers": args.layers} if args.layers else {}
        cfg = wall_oss_config(action_expert_intermediate=args.action_ffn, **cfg_kw)
        proc = make_processor(cfg, 2048)
        torch.manual_seed(1234)
        old = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        with torch.device(dev):
            model = Qwen2_5_VLMoEForAction(cfg, processor=proc, use_fast_tokenizer=(mode == "fast"))
        torch.set_default_dtype(old)
        model.train()
        self.cfg, self.model = cfg, model
        self.accum = max(1, args.per_gpu_batch // args.micro_batch)
        self.micro = args.per_gpu_batch // self.accum
        transport = args.transport
        if transport == "auto":
            transport = "symm" if world > 1 else "local"
        self.transport = transport if world > 1 else "local"
        symm = symm_factory() if self.transport == "symm" else None
        self.engine = TrainEngine(model, lr=9e-5, weight_decay=0.1, max_grad_norm=1.0, grad_accum=self.accum, world=world,
                                  rank=rank, transport=self.transport, symm=symm, shard_params=shard)
        self.engine.overlap_reduce = (world > 1 and self.transport == "symm" and not args.no_overlap_reduce)
        # every rank sees the same modalities in every batch here, so the per-step agreement on which
        # parameters received a gradient (one small all-reduce and a host read) is not needed
        self.engine.check_touched = False
        self.n_params = sum(b.numel for b in self.engine.buffers)
        # ---- synthetic data: a small pool of distinct global batches, pinned on the host
        gen = torch.Generator().manual_seed(100 + rank)
        self.pool = []
        for _ in range(2):
            mbs = []
            for _a in range(self.accum):
                b = make_batch(cfg, proc, self.micro, views=3, image_hw=(256, 256), prompt_len=64, horizon=32, mode=mode,
                               fast_tokens=48, generator=gen, raw_images=True)
                mbs.append(pin_batch(add_pack_info(b, cfg)))
            self.pool.append(mbs)
        vc = cfg.vision_config

        def stage(b_host):
            """Host (pinned) -> device copy of one micro-batch, then patchify on the device."""
            b = to_device(b_host, dev, torch.bfloat16, non_blocking=True)
            imgs = b.pop("images_uint8")
            pv, _ = images_to_patches(imgs, vc.patch_size, vc.temporal_patch_size, vc.spatial_merge_size, torch.bfloat16)
            b["pixel_values"] = pv
            return b

        self.stage = stage
        self.resident = [[stage(b) for b in mbs] for mbs in self.pool]
        torch.cuda.synchronize()

    def h2d_bytes(self):
        import torch

        return sum(v.numel() * v.element_size() for b in self.pool[0] for k, v in b.items()
                   if isinstance(v, torch.Tensor) and k != "seq_lens")

    def train_step(self, mbs_dev):
        loss = None
        for mb in mbs_dev:
            out = self.model(mode="train", **mb)
            self.engine.backward(out.loss)
            loss = out.loss.detach()
        self.engine.optimizer_step(9e-5)
        return loss

    def barrier(self):
        import torch
        import torch.distributed as dist

        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(self, steps: int, warmup: int, e2e: bool = False):
        """(ms per step on the device, host enqueue ms per step, last loss). ``e2e``: every step copies its inputs
        from pinned host memory and reads the loss back."""
        import torch

        from wallx_b200.ops import gemm as G

        for i in range(warmup):
            self.train_step([self.stage(b) for b in self.pool[i % len(self.pool)]] if e2e else self.resident[i % len(self.resident)])
        self.barrier()
        G.check_status()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t0 = time.perf_counter()
        loss = None
        for i in range(steps):
            if e2e:
                loss = self.train_step([self.stage(b) for b in self.pool[i % len(self.pool)]])
                _ = loss.float().cpu()  # device -> host read of the step's result
            else:
                loss = self.train_step(self.resident[i % len(self.resident)])
        host_ms = (time.perf_counter() - t0) * 1e3 / steps
        e1.record()
        self.barrier()
        ms = e0.elapsed_time(e1)
        G.check_status()
        self.engine.check_status()
        # a plain float: the loss tensor's autograd graph would keep every parameter (and with it the whole engine) alive
        return ms, host_ms, float(loss.item())

    def host_ms_per_step(self, steps: int = 3) -> float:
        """Host time to enqueue one full step (all launches of forward, backward and optimizer). Measured at
        micro-batch 2: the number of launches is the same as at the benchmark's batch, but the device finishes each
        kernel faster than the host issues the next one, so the wall time of the loop IS the host time. (At the real
        batch the launch queue fills up and the host just waits for the device, so timing the loop there measures the
        device.)"""
        import torch

        from wallx_b200.data.collator import add_pack_info, pin_batch
        from wallx_b200.data.synthetic import make_batch, make_processor

        gen = torch.Generator().manual_seed(7)
        proc = make_processor(self.cfg, 2048)
        small = [self.stage(pin_batch(add_pack_info(
            make_batch(self.cfg, proc, 2, views=3, image_hw=(256, 256), prompt_len=64, horizon=32, mode=self.mode,
                       fast_tokens=48, generator=gen, raw_images=True), self.cfg))) for _ in range(self.accum)]
        for _ in range(2):
            self.train_step(small)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            self.train_step(small)
        host = (time.perf_counter() - t0) * 1e3 / steps
        torch.cuda.synchronize()
        return host

    def parallelism(self):
        w, tr = self.world, self.transport
        ov = ", reduce-scatter overlapped with backward" if self.engine.overlap_reduce else ""
        if self.shard:
            return (f"fsdp{w} / ZeRO-3 (layer weights stored as rows per GPU, all-gather fused into the forward and dgrad "
                    f"GEMMs, bf16 wgrad reduce-scattered by peer loads, AdamW on the owner's rows; transport={tr}{ov})")
        return f"dp{w} (resident bf16 params; sharded fp32 master + Adam moments; transport={tr}{ov})"

    def close(self):
        import gc

        import torch

        from wallx_b200.ops import functional as F_

        F_.clear_grad_sinks()
        self.engine.close()
        self.engine = self.model = self.resident = self.pool = self.stage = None
        gc.collect()
        torch.cuda.empty_cache()


def max_over_ranks(vals, dev, world):
    import torch
    import torch.distributed as dist

    t = torch.tensor(list(vals), device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


def latency_block(args, world, rank, dev):
    """p50 / p99 of one flow action chunk (H2D of the observation .. D2H of the 32 x 20 chunk, 10 Euler evaluations
    on the cached prefix), batch 1 and 32, model replicated on every rank, max over ranks."""
    import torch

    from wallx_b200.bench.flow_latency import _percentile, _pin
    from wallx_b200.config import wall_oss_config
    from wallx_b200.data.synthetic import make_batch, make_processor
    from wallx_b200.models import Qwen2_5_VLMoEForAction
    from wallx_b200.models.inference import FlowEngine

    cfg = wall_oss_config(action_expert_intermediate=args.action_ffn, **({"num_hidden_layers": args.layers} if args.layers else {}))
    proc = make_processor(cfg, 2048)
    torch.manual_seed(1234)
    model = Qwen2_5_VLMoEForAction(cfg, processor=proc).to(torch.bfloat16).to(dev)
    model.init_weights(seed=0)
    model.eval()
    out = {"unit": "ms per chunk", "euler_evaluations": 10, "chunks": args.latency_chunks,
           "path": "FlowEngine: prefix pass + 10 evaluations in one CUDA graph; timed H2D of the observation to D2H of the chunk"}
    for B in (1, 32):
        gen = torch.Generator().manual_seed(100 + rank)
        pool = []
        for _ in range(3):
            b = make_batch(cfg, proc, B, views=3, image_hw=(256, 256), prompt_len=64, horizon=32, mode="flow", generator=gen)
            b.pop("action_chunk", None)
            b.pop("labels", None)
            pool.append(_pin(b))
        engine = FlowEngine(model, pool[0], num_inference_timesteps=10)
        for i in range(3):
            engine(pool[i % 3])["predict_action"].float().cpu()
        torch.cuda.synchronize()
        times = []
        for i in range(args.latency_chunks):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine(pool[i % 3])["predict_action"].float().cpu()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        p50, p99 = max_over_ranks([_percentile(times, 0.5), _percentile(times, 0.99)], dev, world)
        out[f"batch{B}"] = {"p50_ms": round(p50, 3), "p99_ms": round(p99, 3)}
        del engine
    return out


def main():
    args = parse()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():  # the training step is CUDA kernels only: no CPU fallback is timed
        print(json.dumps({"impl": "ours", "unavailable": "no CUDA device: this benchmark needs a B200"}), flush=True)
        sys.exit(1)

    from wallx_b200.ops import _ext

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"

    comm = []

    def symm_factory():  # one transport object for all arms: its symmetric arenas are reused, not re-allocated
        from wallx_b200.parallel.symm import SymmComm

        if not comm:
            comm.append(SymmComm(dist.group.WORLD, dev))
        return comm[0]

    arm = Arm(args, args.mode, args.shard_params, world, rank, dev, symm_factory)
    # ---- warm-up, then timed: device-resident inputs
    for i in range(args.warmup):
        arm.train_step(arm.resident[i % len(arm.resident)])
    arm.barrier()
    counter = _ext.LaunchCounter.install()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_dev, host_ms, loss = arm.timed(args.steps, 0)
    launches = counter.total
    counter.uninstall()
    clocks = sampler.stop() if rank == 0 else None
    loss_val = loss
    # ---- timed: end to end (pinned host -> device every step, loss read back every step)
    ms_e2e = None
    if not args.no_e2e:
        ms_e2e, _, _ = arm.timed(args.steps, 1, e2e=True)
    host_only = arm.host_ms_per_step()
    ms_dev, ms_e2e_max, host_only = max_over_ranks([ms_dev, ms_e2e if ms_e2e is not None else 0.0, host_only], dev, world)
    global_batch = args.per_gpu_batch * world
    def peak_memory_gb(a):
        # caching-allocator peak plus the symmetric arenas (bf16 parameters / shards and gradients at N > 1), which
        # the allocator does not see
        sym = a.engine.symm.arena_bytes() if a.engine.symm is not None else 0
        return max_over_ranks([(torch.cuda.max_memory_allocated(dev) + sym) / 2 ** 30], dev, world)[0]

    peak_gb = peak_memory_gb(arm)
    rec = {
        "metric": f"train samples/s, WALL-OSS-{args.mode.upper()}-size fine-tune (max over ranks, device-timed)",
        "value": round(global_batch * args.steps / (ms_dev / 1e3), 3), "unit": "samples/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_dev / args.steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": f"WALL-OSS-{args.mode.upper()} (Qwen2.5-VL-3B backbone, 36 layers, action expert FFN {args.action_ffn}, ViT 32 blocks)"
                     + (f" DEBUG layers={args.layers}" if args.layers else ""),
            "global_batch": global_batch, "per_gpu_batch": args.per_gpu_batch, "micro_batch": arm.micro,
            "grad_accum": arm.accum, "seq_len": int(arm.pool[0][0]["input_ids"].shape[1]),
            "vit_patches_per_sample": 3 * 18 * 18, "params": arm.n_params, "parallelism": arm.parallelism(),
            "optimizer": "fused AdamW, wd 0.1, clip 1.0, fp32 master",
            "host_enqueue_ms_per_step": round(host_only, 1),
            "host_enqueue_note": "host time to issue one step's launches, measured at micro-batch 2 where the device is not the limiter; "
                                 f"the loop at the benchmark batch took {round(host_ms, 1)} ms/step of wall time, i.e. it waits for the device",
            "peak_device_memory_gb": round(peak_gb, 1),
            "l2_policy": "inputs and weights (>8 GB) are far larger than L2; no explicit flush",
            "loss": loss_val,
        },
        "clocks": clocks, "gpu_launches": int(launches),
    }
    if ms_e2e is not None:
        rec["e2e"] = {"value": round(global_batch * args.steps / (ms_e2e_max / 1e3), 3), "unit": "samples/s",
                      "h2d_bytes_per_step": int(arm.h2d_bytes()), "d2h_bytes_per_step": 4,
                      "ms_per_step": round(ms_e2e_max / args.steps, 3)}
    if args.kernel_table and rank == 0:
        write_kernel_table(args.kernel_table, lambda: arm.train_step(arm.resident[0]))
    arm.close()

    # ---- further measurements, all outside the headline timed region (short: few steps each)
    def extra(name, fn):
        try:
            rec[name] = fn()
        except Exception as e:  # an extra block never takes the headline down
            import traceback

            traceback.print_exc(file=sys.stderr)
            rec[name] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
        if world > 1:
            dist.barrier()

    def train_block(mode, shard):
        torch.cuda.reset_peak_memory_stats(dev)
        a = Arm(args, mode, shard, world, rank, dev, symm_factory)
        k = max(2, min(args.steps, args.extra_steps))
        ms, host, l = a.timed(k, 2)
        ms = max_over_ranks([ms], dev, world)[0]
        pk = peak_memory_gb(a)
        out = {"value": round(global_batch * k / (ms / 1e3), 3), "unit": "samples/s", "ms_per_step": round(ms / k, 3),
               "steps": k, "warmup": 2, "n_gpus": world, "peak_device_memory_gb": round(pk, 1),
               "host_enqueue_ms_per_step": round(host, 1), "parallelism": a.parallelism(), "loss": l}
        a.close()
        return out

    if not args.no_extras:
        other = not args.shard_params
        extra("zero3" if other else "resident", lambda: train_block(args.mode, other))
        if args.mode == "flow":
            extra("fast", lambda: train_block("fast", args.shard_params))
        extra("latency", lambda: latency_block(args, world, rank, dev))
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.destroy_process_group()


def write_kernel_table(path, step_fn):
    """Trace ONE extra step (outside every timed region) and write each kernel's share of the
    device time. Shares only: absolute times under the tracer are not benchmark numbers."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step_fn()
        torch.cuda.synchronize()
    rows = []
    for ev in prof.key_averages():
        t = getattr(ev, "self_device_time_total", None)
        if t is None:
            t = getattr(ev, "self_cuda_time_total", 0.0)
        if t > 0:
            rows.append((ev.key, int(ev.count), float(t)))
    rows.sort(key=lambda r: -r[2])
    total = sum(r[2] for r in rows) or 1.0
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    with open(path, "w") as f:
        f.write(f"# one training step, kernel time shares (sum of kernel time {total / 1e3:.1f} ms under the tracer)\n")
        f.write(f"# {'share':>6} {'ms':>9} {'calls':>6}  kernel\n")
        for name, n, t in rows[:60]:
            f.write(f"  {100 * t / total:6.2f} {t / 1e3:9.3f} {n:6d}  {name[:150]}\n")


if __name__ == "__main__":
    main()

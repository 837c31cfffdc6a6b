"""Trainer, engine, optimizer sharding, checkpoint resharding and failure handling on CPU (gloo)."""
import copy
import json
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from wallx_b200.config import tiny_config
from wallx_b200.data.collator import add_pack_info
from wallx_b200.data.synthetic import make_batch, make_processor
from wallx_b200.models import Qwen2_5_VLMoEForAction
from wallx_b200.parallel.engine import TrainEngine, default_units
from wallx_b200.train.schedule import CosineWithMinLR


def _model(seed=0):
    cfg = tiny_config()
    proc = make_processor(cfg, 16)
    m = Qwen2_5_VLMoEForAction(cfg, processor=proc)
    m.init_weights(seed=seed)
    return cfg, proc, m


def _batches(cfg, proc, n, B=2, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        b = add_pack_info(make_batch(cfg, proc, B, views=1, image_hw=(112, 112), prompt_len=16, horizon=16, generator=g), cfg)
        b["flow_noise"] = torch.randn(b["action_chunk"].shape, generator=g)
        b["flow_time"] = torch.rand(B, generator=g)
        out.append(b)
    return out


def test_schedule_matches_closed_form():
    s = CosineWithMinLR(1e-3, 10, 110, min_lr=1e-4)
    assert s.get_lr() == 0.0
    for _ in range(10):
        s.step()
    assert abs(s.get_lr() - 1e-3) < 1e-12
    for _ in range(50):
        s.step()
    assert abs(s.get_lr() - (1e-4 + (1e-3 - 1e-4) * 0.5)) < 1e-9
    for _ in range(50):
        s.step()
    assert abs(s.get_lr() - 1e-4) < 1e-9


def test_units_cover_every_trainable_parameter_once():
    _, _, m = _model()
    units = default_units(m)
    names = [n for _, ps in units for n, _ in ps]
    assert len(names) == len(set(names))
    assert sum(p.numel() for _, ps in units for _, p in ps) == sum(p.numel() for p in m.parameters() if p.requires_grad)
    assert [u for u, _ in units][:2] == ["visual.blocks.0", "visual.blocks.1"] and units[-1][0] == "root"


def test_engine_step_matches_torch_adamw_with_clipping():
    cfg, proc, m = _model()
    ref_m = copy.deepcopy(m)
    eng = TrainEngine(m, lr=1e-3, weight_decay=0.1, max_grad_norm=0.5, grad_accum=2)
    opt = torch.optim.AdamW([p for p in ref_m.parameters() if p.requires_grad], lr=1e-3, weight_decay=0.1)
    for step in range(2):
        bs = _batches(cfg, proc, 2, seed=step)
        for b in bs:
            eng.backward(m(mode="train", **b).loss)
            (ref_m(mode="train", **b).loss / 2).backward()
        torch.nn.utils.clip_grad_norm_([p for p in ref_m.parameters() if p.requires_grad], 0.5)
        opt.step()
        opt.zero_grad()
        eng.optimizer_step(1e-3)
    for (n, a), (_, b) in zip(m.named_parameters(), ref_m.named_parameters()):
        assert torch.allclose(a, b, atol=2e-6), n
    assert eng.grad_norm().item() > 0


def test_nonfinite_gradient_skips_the_update_everywhere():
    cfg, proc, m = _model()
    eng = TrainEngine(m, lr=1e-3, grad_accum=1)
    before = eng.buffers[0].param.clone()
    eng.backward(m(mode="train", **_batches(cfg, proc, 1)[0]).loss)
    eng.buffers[3].grad[5] = float("nan")
    eng.optimizer_step(1e-3)
    assert torch.equal(eng.buffers[0].param, before)  # no buffer moved, not just the poisoned one
    assert eng.buffers[3].grad.abs().sum() == 0  # gradients were still cleared


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _dist_worker(rank, world, port, tmp, mode):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.distributed.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    cfg, proc, m = _model()
    eng = TrainEngine(m, lr=1e-3, weight_decay=0.1, max_grad_norm=1.0, grad_accum=1, world=world, rank=rank, transport="dist")
    all_b = _batches(cfg, proc, 2 * world, seed=3)
    if mode == "peer_never_joins" and rank == 1:
        torch.distributed.destroy_process_group()
        return
    for step in range(2):
        b = all_b[step * world + rank]
        eng.backward(m(mode="train", **b).loss)
        if mode == "rank_raises" and step == 1 and rank == 1:
            raise RuntimeError("injected failure on rank 1")
        eng.optimizer_step(1e-3)
    torch.save({n: p.detach().clone() for n, p in m.named_parameters()}, os.path.join(tmp, f"params_{rank}.pt"))
    torch.save(eng.optimizer_state(), os.path.join(tmp, f"optim_rank{rank:05d}_of_{world:05d}.pt"))
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world", [2, 4])
def test_gloo_training_equals_single_rank_large_batch(tmp_path, world):
    mp.spawn(_dist_worker, args=(world, _free_port(), str(tmp_path), "ok"), nprocs=world, join=True)
    p0 = torch.load(tmp_path / "params_0.pt")
    for r in range(1, world):
        pr = torch.load(tmp_path / f"params_{r}.pt")
        for k in p0:
            assert torch.equal(p0[k], pr[k]), k  # replicas stay identical
    # single process, every rank's micro-batch per step (== data parallel average)
    cfg, proc, m = _model()
    eng = TrainEngine(m, lr=1e-3, weight_decay=0.1, max_grad_norm=1.0, grad_accum=world)
    all_b = _batches(cfg, proc, 2 * world, seed=3)
    for step in range(2):
        for r in range(world):
            eng.backward(m(mode="train", **all_b[step * world + r]).loss)
        eng.optimizer_step(1e-3)
    for n, p in m.named_parameters():
        assert torch.allclose(p, p0[n], atol=3e-5), n  # 3% of one lr-sized Adam step: rounding only
    # reshard the sharded optimizer state onto 1 rank and compare with the single-rank state
    from wallx_b200.parallel.reshard import load_optimizer_shards

    cfg, proc, m2 = _model()
    eng2 = TrainEngine(m2, lr=1e-3, grad_accum=1)
    load_optimizer_shards(eng2, str(tmp_path), world)
    assert eng2.optimizer.step_count == 2
    for a, b in zip(eng.buffers, eng2.buffers):
        assert torch.allclose(a.exp_avg[: a.numel], b.exp_avg[: b.numel], atol=1e-6)
        assert torch.allclose(a.master[: a.numel], b.master[: b.numel], atol=3e-5)


@pytest.mark.timeout(300)
def test_rank_failure_is_reported_not_hung(tmp_path):
    """A rank that raises between steps takes the job down with an error instead of a hang."""
    with pytest.raises(Exception):
        mp.spawn(_dist_worker, args=(2, _free_port(), str(tmp_path), "rank_raises"), nprocs=2, join=True)


def test_watchdog_raises_after_timeout():
    import time

    from wallx_b200.train.trainer import StepWatchdog

    w = StepWatchdog(0.05)
    w.check()
    time.sleep(0.1)
    with pytest.raises(TimeoutError):
        w.check()
    w.kick()
    w.check()


def test_trainer_fit_save_resume(tmp_path):
    from wallx_b200.train.trainer import QwenVlAct_Trainer

    config = {
        "model": {"preset": "tiny"}, "save_path": str(tmp_path / "run"), "learning_rate": 1e-3, "min_lr": 1e-4,
        "num_warmup_steps": 1, "num_training_steps": 10, "num_epoch": 1, "gradient_accumulation_steps": 2,
        "batch_size_per_gpu": 2, "num_workers": 0, "epoch_save_interval": 1, "max_steps": 3,
        "data": {"synthetic": True, "action_horizon": 16, "synthetic_config": {"num_samples": 20, "image_hw": [112, 112]},
                 "resolution": {"face_view": 112, "left_wrist_view": 112, "right_wrist_view": 112}},
    }
    tr = QwenVlAct_Trainer(config, seed=1)
    tr.fit()
    assert tr.global_step == 3
    ck = tmp_path / "run" / "0"
    assert (ck / "config.json").exists() and (ck / "model.safetensors").exists() and (ck / "trainer_state.json").exists()
    lines = [json.loads(l) for l in open(tmp_path / "run" / "metrics.jsonl")]
    assert any("train_loss" in l and "flow_loss" in l and "total_norm" in l and "lr" in l for l in lines)
    assert any("val_loss" in l for l in lines)
    config2 = dict(config, resume={"ckpt": str(ck)}, num_epoch=2, max_steps=4)
    tr2 = QwenVlAct_Trainer(config2, seed=1)
    assert tr2.global_step == 3 and tr2.epoch == 1 and tr2.lr_scheduler.step_count == 3
    for a, b in zip(tr.engine.buffers, tr2.engine.buffers):
        assert torch.equal(a.exp_avg, b.exp_avg) and torch.allclose(a.master, b.master, atol=1e-6)
    sd1, sd2 = tr.model.state_dict(), tr2.model.state_dict()
    assert all(torch.equal(sd1[k], sd2[k]) for k in sd1)


def test_timers_accumulate_and_log(capsys):
    import time

    from wallx_b200.utils.timers import Timers

    t = Timers(log_level=0, log_option="minmax")
    t("fwd", 0).start()
    time.sleep(0.02)
    t("fwd", 0).stop()
    t("skipped", 2).start()  # above the log level: a no-op dummy
    t.log(["fwd"])
    out = capsys.readouterr().out
    assert "fwd" in out and "(min, max)" in out
    assert t("fwd", 0).elapsed() == 0.0


def test_example_yaml_has_every_trainer_key():
    """The shipped fine-tuning YAML parses through the CLI loader and carries every key without a default."""
    import os

    import train_qact

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = train_qact.load_config(os.path.join(root, "workspace", "lerobot_example", "finetune_flow.yml"))
    for key in ("pretrained_wallx_path", "save_path", "learning_rate", "min_lr", "num_warmup_steps", "num_training_steps",
                "num_epoch", "gradient_accumulation_steps", "batch_size_per_gpu", "dof_config", "agent_pos_config", "data"):
        assert key in cfg, key
    assert cfg["data"]["model_type"] == "qwen2_5"
    assert cfg["dof_config"] == cfg["agent_pos_config"] and sum(cfg["dof_config"].values()) == 20
    d = cfg["data"]
    assert d["action_horizon"] == 32 and d["obs_action_keys"] == d["predict_action_keys"] == list(cfg["dof_config"])
    assert d["lerobot_config"]["repo_id"] == "lerobot/aloha_mobile_cabinet" and d["resolution"]["face_view"] == 256
    from wallx_b200.data.lerobot import get_data_configs

    assert get_data_configs(d)["action_horizon"] == 33


def test_timer_active_time_survives_reset_and_collator_normalize():
    import time

    from wallx_b200.data.collator import DataCollator, minmax_normalize
    from wallx_b200.utils.timers import DummyTimer, Timer

    t = Timer("t", use_cuda_events=False)
    for _ in range(2):
        t.start()
        time.sleep(0.01)
        t.stop()
        assert t.elapsed(reset=True) >= 0.009
    assert t.active_time() >= 0.018 and t.elapsed(reset=False) == 0.0
    with pytest.raises(RuntimeError):
        DummyTimer().active_time()
    x = torch.tensor([[0.0, 5.0, 10.0], [2.0, 5.0, 20.0]])
    mn, mx = [0.0, 5.0, 0.0], [4.0, 5.0, 10.0]
    a = DataCollator._normalize(x, mn, [4.0, 0.0, 10.0])
    assert torch.equal(a, minmax_normalize(x, mn, mx))
    assert a.tolist() == [[-1.0, -1.0, 1.0], [0.0, -1.0, 1.0]]  # zero range counts as 1; values are clamped


def test_nvtx_annotation_is_off_by_default_and_wraps_on_request(monkeypatch):
    import types

    from wallx_b200.ops import functional as F_
    from wallx_b200.utils import nvtx

    assert not nvtx.enabled() and not getattr(F_.linear, "__wrapped_by_nvtx__", False)  # default: untouched call path
    mod = types.SimpleNamespace(f=lambda x: x + 1, g=3)
    assert nvtx.annotate_module(mod, ["f", "g"]) == 0
    monkeypatch.setenv("WALLX_NVTX", "1")
    assert nvtx.annotate_module(mod, ["f", "g", "missing"]) == 1
    assert mod.f(1) == 2 and mod.f.__wrapped_by_nvtx__  # on a CPU box the range calls are skipped
    assert nvtx.annotate_module(mod, ["f"]) == 0  # idempotent
    for name in F_.NVTX_OPS:
        assert callable(getattr(F_, name)), name


def test_corrupt_or_missing_checkpoint_files_raise_cleanly(tmp_path):
    """Host-side fault injection on checkpoint files: a truncated optimizer shard and an empty weights directory."""
    from wallx_b200.parallel.reshard import load_optimizer_shards
    from wallx_b200.train import checkpoint as CK

    m = torch.nn.Sequential(torch.nn.Linear(8, 8))
    eng = TrainEngine(m, lr=1e-3)
    f = tmp_path / "optim_rank00000_of_00001.pt"
    torch.save(eng.optimizer_state(), f)
    load_optimizer_shards(eng, str(tmp_path), 1)  # intact: loads
    data = f.read_bytes()
    f.write_bytes(data[: len(data) // 2])
    with pytest.raises(Exception):
        load_optimizer_shards(eng, str(tmp_path), 1)
    with pytest.raises(FileNotFoundError):
        CK.load_safetensors_dir(str(tmp_path / "nothing_here"))
    # a checkpoint of another model is refused instead of being half-loaded
    m2 = torch.nn.Sequential(torch.nn.Linear(8, 9))
    torch.save(TrainEngine(m2, lr=1e-3).optimizer_state(), f)
    with pytest.raises(ValueError):
        load_optimizer_shards(eng, str(tmp_path), 1)


def _zero3_worker(rank, world, port, tmp, clip):
    """Resident-parameter engine and row-sharded (ZeRO-3) engine on the same model, data and ranks."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.distributed.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    out = {}
    for plan in ("resident", "sharded"):
        cfg, proc, m = _model()
        eng = TrainEngine(m, lr=1e-3, weight_decay=0.1, max_grad_norm=clip, grad_accum=2, world=world, rank=rank,
                          transport="dist" if world > 1 else "local", shard_params=(plan == "sharded"))
        if plan == "sharded":
            rows = [b for b in eng.buffers if b.kind == "rows"]
            assert len(rows) == cfg.num_hidden_layers + cfg.vision_config.depth and eng.buffers[-1].kind == "flat"
            for b in rows:  # every rank owns rows [rank * R / world, (rank + 1) * R / world) of every weight of the unit
                assert b.shard_numel * world == b.numel and all(p.dim() == 2 for p in b.params)
        all_b = _batches(cfg, proc, 4 * world, seed=3)
        norms = []
        for step in range(2):
            for a in range(2):
                eng.backward(m(mode="train", **all_b[(step * 2 + a) * world + rank]).loss)
            eng.optimizer_step(1e-3)
            norms.append(eng.grad_norm().item())
        with eng.gathered_parameters():
            out[plan] = {n: p.detach().clone() for n, p in m.named_parameters()}
        out[plan + "_norms"] = norms
        if plan == "sharded":
            torch.save(eng.optimizer_state(), os.path.join(tmp, f"optim_rank{rank:05d}_of_{world:05d}.pt"))
            if rank == 0:
                with eng.gathered_parameters():
                    m.save_pretrained(os.path.join(tmp, "export"))
            # writing whole weights back into the shards (resume path): perturb, write back, read again
            with eng.gathered_parameters(writeback=True):
                for p in m.parameters():
                    p.data.add_(1.0)
            with eng.gathered_parameters():
                for n, p in m.named_parameters():
                    assert torch.allclose(p, out[plan][n] + 1.0, atol=1e-6), n
            for b in eng.buffers:
                s0, s1 = b.shard_range
                assert torch.equal(b.master, b.param[s0:s1].to(b.master.dtype))
    torch.save(out, os.path.join(tmp, f"z3_{rank}.pt"))
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_row_sharded_parameters_train_like_resident_ones(tmp_path, world):
    """ZeRO-3 storage (rows of every weight per rank, whole-gradient reduction onto the owner's rows, AdamW on the
    rows, refresh by collective) gives bit-identical parameters to the resident plan when no clipping interferes:
    the same elements are reduced and updated, only their owner differs. The optimizer state reshards by name."""
    mp.spawn(_zero3_worker, args=(world, _free_port(), str(tmp_path), 1e9), nprocs=world, join=True)
    outs = [torch.load(tmp_path / f"z3_{r}.pt") for r in range(world)]
    for r in range(world):
        for k, v in outs[0]["resident"].items():
            got = outs[r]["sharded"][k]
            if world <= 2:
                assert torch.equal(got, v), (r, k)
            else:
                # gloo's ring all-reduce adds the ranks in an order that depends on where an element sits in the
                # reduced buffer, and the two plans lay the buffers out differently: with more than two ranks the
                # sums differ in the last bit, which Adam turns into lr-sized steps where the true gradient is ~0
                assert torch.equal(got, outs[0]["sharded"][k]), (r, k)  # replicas identical
                assert torch.allclose(got, v, atol=2.5e-3), (r, k)
                assert ((got - v).abs() > 1e-5).float().mean() < 0.05, (r, k)  # 1e-5 = 1 % of one lr-sized step
        assert outs[r]["sharded_norms"] == pytest.approx(outs[0]["resident_norms"], rel=1e-5)
    # the optimizer state of the sharded run, resharded onto one rank of either plan, equals a single-rank run
    from wallx_b200.parallel.reshard import load_optimizer_shards

    cfg, proc, m = _model()
    eng = TrainEngine(m, lr=1e-3, weight_decay=0.1, max_grad_norm=1e9, grad_accum=2 * world)
    all_b = _batches(cfg, proc, 4 * world, seed=3)
    threads = torch.get_num_threads()
    torch.set_num_threads(1)  # as the workers: Adam turns summation-order noise in near-zero gradients into lr-sized steps
    try:
        for step in range(2):
            for a in range(2):
                for r in range(world):
                    eng.backward(m(mode="train", **all_b[(step * 2 + a) * world + r]).loss)
            eng.optimizer_step(1e-3)
    finally:
        torch.set_num_threads(threads)
    for shard in (False, True):
        cfg, proc, m2 = _model()
        eng2 = TrainEngine(m2, lr=1e-3, grad_accum=1, shard_params=shard)
        load_optimizer_shards(eng2, str(tmp_path), world)
        assert eng2.optimizer.step_count == 2
        got = {n: (b.exp_avg[o:o + p.numel()], b.master[o:o + p.numel()])
               for b in eng2.buffers for n, p, o in zip(b.names, b.params, b.offsets)}
        want = {n: (b.exp_avg[o:o + p.numel()], b.master[o:o + p.numel()])
                for b in eng.buffers for n, p, o in zip(b.names, b.params, b.offsets)}
        assert set(got) == set(want)
        for n in want:
            assert torch.allclose(got[n][0], want[n][0], atol=1e-6), n
            assert torch.allclose(got[n][1], want[n][1], atol=3e-5), n
    # the exported checkpoint holds whole weights under the reference's key names
    from wallx_b200.train.checkpoint import load_safetensors_dir

    state = load_safetensors_dir(str(tmp_path / "export"))
    cfg, proc, m3 = _model()
    missing, unexpected = m3.load_state_dict(state, strict=False)
    assert not unexpected and all("normalizer" in k or "inv_freq" in k for k in missing), (missing, unexpected)
    for n, p in m3.named_parameters():
        assert torch.allclose(p, outs[0]["sharded"][n], atol=1e-6), n


@pytest.mark.timeout(600)
def test_row_sharded_parameters_with_clipping_over_gloo(tmp_path):
    """With clipping active the two plans differ only through the summation order of the squared norm."""
    mp.spawn(_zero3_worker, args=(2, _free_port(), str(tmp_path), 0.5), nprocs=2, join=True)
    o = torch.load(tmp_path / "z3_0.pt")
    for k, v in o["resident"].items():
        assert torch.allclose(o["sharded"][k], v, atol=1e-6), k
    assert o["sharded_norms"] == pytest.approx(o["resident_norms"], rel=1e-5)


def test_accumulation_remainder_and_early_announcement_are_reduced_correctly(monkeypatch):
    """Host logic of gradient accumulation against the fake transport: (a) a backward that arrives after units were
    reduced early makes every unit be reduced again; (b) a step after fewer micro-batches than configured averages over
    the true count."""
    torch.manual_seed(0)
    m = _two_layer_wrapper()
    fake = _FakeSymm()
    eng = TrainEngine(m, lr=1e-2, weight_decay=0.0, max_grad_norm=0.0, grad_accum=2, world=2, rank=0, transport="symm", symm=fake)
    eng.overlap_reduce = True
    eng.check_touched = False
    monkeypatch.setattr(eng, "_early_reduce", lambda k: (fake.reduce_scatter_unit(k), eng._early.add(k)))
    x = torch.randn(4, 6)

    def micro(last=None):
        eng.backward(m(x).pow(2).mean(), last=last)

    micro(), micro(), eng.optimizer_step(1e-2)  # learns the triggers
    fake.calls.clear()
    micro(last=True)   # announced too early: units get reduced during this backward ...
    early = [c for c in fake.calls if isinstance(c, int)]
    assert early, "units should have been reduced during the backward that was announced as the last one"
    micro(last=True)   # ... but another micro-batch follows: everything is reduced again
    g_full = [b.grad.clone() for b in eng.buffers]
    eng.optimizer_step(1e-2)
    begins = [i for i, c in enumerate(fake.calls) if c == "begin"]
    after_last_begin = [c for c in fake.calls[begins[-1]:] if isinstance(c, int)]
    assert sorted(after_last_begin) == list(range(len(eng.buffers)))
    for k, b in enumerate(eng.buffers):  # the reduced shard is the whole accumulated gradient (own + identical peer)
        s0, s1 = b.shard_range
        assert torch.allclose(fake._shards_seen[k], 2.0 * g_full[k][s0:s1].float())
    # (b) one micro-batch only, then step: scale 1 / (1 * world), not 1 / (2 * world)
    micro(last=True)
    eng.optimizer_step(1e-2)
    assert eng.optimizer.grad_accum == 1 * 2 and eng._last_micro == 1


def test_timed_out_device_wait_skips_the_step_on_every_rank_and_raises():
    """A non-zero status word of the transport (a barrier that gave up) poisons the all-reduced norm, so the update is
    skipped everywhere, and the host check raises."""
    eng = TrainEngine(torch.nn.Linear(4, 4), lr=1e-2, grad_accum=1)
    eng.last_bad = torch.ones(1)
    with pytest.raises(RuntimeError, match="timed out"):
        eng.check_status()
    eng.check_status()  # cleared
    # the poison itself: a non-finite norm leaves parameters untouched (same rule as a non-finite gradient)
    m = torch.nn.Linear(4, 4)
    eng = TrainEngine(m, lr=1e-2, grad_accum=1)
    before = m.weight.detach().clone()
    eng.backward(m(torch.randn(3, 4)).sum())
    orig = eng._global_norm_sq
    eng._global_norm_sq = lambda shards: orig(shards).fill_(float("nan"))
    eng.optimizer_step(1e-2)
    assert torch.equal(m.weight.detach(), before)


def test_typed_training_config_accepts_the_example_and_names_bad_keys():
    import yaml

    from wallx_b200.train.config import TrainConfig

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "workspace", "lerobot_example", "finetune_flow.yml")) as f:
        raw = yaml.safe_load(f)
    tc = TrainConfig.from_dict(raw).validate(require_paths=True)
    assert tc.unknown_keys == [] and tc.learning_rate == 9e-5 and tc.transport == "auto" and tc.FSDP2 is True
    assert sum(tc.dof_config.values()) == 20 and tc.data["action_horizon"] == 32
    for key, bad, word in [("learning_rate", -1.0, "learning_rate"), ("min_lr", 1.0, "min_lr"), ("batch_size_per_gpu", 0, "batch_size_per_gpu"),
                           ("gradient_accumulation_steps", 1.5, "gradient_accumulation_steps"), ("transport", "tcp", "transport"),
                           ("optimizer_dtype", "fp8", "optimizer_dtype"), ("use_fast_tokenizer", "yes", "use_fast_tokenizer"),
                           ("dof_config", {"arm": 21}, "dof_config"), ("padding_side", "top", "padding_side"),
                           ("resume", {"ckpt": "", "load_ckpt_only": True}, "resume"), ("resume", {"ckpt": "x", "oops": 1}, "resume")]:
        cfg = dict(raw)
        cfg[key] = bad
        with pytest.raises(ValueError, match=word):
            TrainConfig.from_dict(cfg).validate()
    extra = dict(raw, my_note="run 7")
    assert TrainConfig.from_dict(extra).validate().unknown_keys == ["my_note"]
    with pytest.raises(ValueError, match="pretrained_wallx_path"):
        TrainConfig.from_dict(dict(raw, pretrained_wallx_path=None)).validate(require_paths=True)


class _FakeSymm:
    """Stand-in for the NVLink transport: rank 0 of 2 whose peer always contributes the same gradients, so a step must
    equal a single-rank step on the doubled gradient. Records when each unit is reduced."""

    def __init__(self):
        self.calls, self.buffers = [], []
        self.local_sumsq = torch.zeros(1)
        self._shards = {}
        self._shards_seen = {}

    def reserve(self, total, dtype=torch.float32, grad_elems=0):
        self.reserved = total

    def alloc_param(self, n, dtype):
        return torch.zeros(n, dtype=dtype)

    def alloc_grad(self, n, dtype):
        return torch.zeros(n, dtype=dtype)

    def register_buffers(self, buffers):
        self.buffers = list(buffers)

    def begin_step(self):
        self.calls.append("begin")
        self.local_sumsq.zero_()
        self._shards = {}

    def reduce_scatter_unit(self, k):
        b = self.buffers[k]
        s0, s1 = b.shard_range
        g = 2.0 * b.grad[s0:s1].float()  # own + identical peer
        self._shards[k] = g
        self._shards_seen[k] = g.clone()
        self.local_sumsq += (g ** 2).sum()
        self.calls.append(k)

    def reduce_scatter_grads(self, buffers):
        self.begin_step()
        for k in reversed(range(len(buffers))):
            self.reduce_scatter_unit(k)
        return self.grad_shards()

    def grad_shards(self):
        return [self._shards[k] for k in range(len(self.buffers))]

    def all_reduce_scalar(self, t):
        return t * 2.0  # the peer's shard carries the same squared norm

    def all_reduce_vector(self, t):
        return t * 2.0

    def all_gather_params(self, buffers):
        self.calls.append("push")


def _two_layer_wrapper():
    m = torch.nn.Sequential(torch.nn.Linear(6, 6), torch.nn.Tanh(), torch.nn.Linear(6, 3))

    class Wrapper(torch.nn.Module):  # two "decoder layers" + a root unit, as default_units expects
        def __init__(self):
            super().__init__()
            self.model = torch.nn.Module()
            self.model.layers = torch.nn.ModuleList([m[0], m[2]])
            self.scale = torch.nn.Parameter(torch.ones(3))

        def forward(self, x):
            return self.model.layers[1](torch.tanh(self.model.layers[0](x))) * self.scale

    return Wrapper()


def test_overlap_schedule_learns_triggers_and_reduces_units_during_backward(monkeypatch):
    """Host logic of the reduce-scatter overlap: the first step records each unit's gradient order, later steps
    reduce a unit as soon as its last gradient arrived (before backward returns), a unit that was not triggered is
    reduced after backward, and every unit is reduced exactly once per step."""
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(6, 6), torch.nn.Tanh(), torch.nn.Linear(6, 3))

    class Wrapper(torch.nn.Module):  # two "decoder layers" + a root unit, as default_units expects
        def __init__(self):
            super().__init__()
            self.model = torch.nn.Module()
            self.model.layers = torch.nn.ModuleList([m[0], m[2]])
            self.scale = torch.nn.Parameter(torch.ones(3))

        def forward(self, x):
            return self.model.layers[1](torch.tanh(self.model.layers[0](x))) * self.scale

    net = Wrapper()
    fake = _FakeSymm()
    eng = TrainEngine(net, lr=1e-2, weight_decay=0.0, max_grad_norm=1e9, world=2, rank=0, transport="symm", symm=fake)
    assert len(eng.buffers) == 3 and fake.buffers == eng.buffers
    eng.overlap_reduce = True
    eng.check_touched = False
    early = []
    monkeypatch.setattr(eng, "_early_reduce", lambda k: (early.append(k), fake.reduce_scatter_unit(k), eng._early.add(k)))
    x = torch.randn(4, 6)
    # step 1: nothing is known yet -> every unit is reduced after backward
    eng.backward(net(x).sum())
    assert fake.calls == ["begin"] and not early
    eng.optimizer_step(1e-2)
    assert sorted(c for c in fake.calls if isinstance(c, int)) == [0, 1, 2] and fake.calls[-1] == "push"
    assert eng._learned and set(eng._trigger) == {0, 1, 2} and all(eng._expected[k] >= 1 for k in range(3))
    # step 2: units whose last gradient is an autograd hook are reduced during backward, in backward order
    fake.calls.clear()
    eng.backward(net(x).sum())
    during = [c for c in fake.calls if isinstance(c, int)]
    assert during == early and len(during) >= 2 and during.index(1) < during.index(0)  # the later layer finishes first
    eng.optimizer_step(1e-2)
    ints = [c for c in fake.calls if isinstance(c, int)]
    assert sorted(ints) == [0, 1, 2]  # each unit exactly once, the rest after backward
    # a step whose backward bypasses engine.backward() is still reduced, just without overlap
    fake.calls.clear()
    early.clear()
    net(x).sum().backward()
    eng.optimizer_step(1e-2)
    assert not early and sorted(c for c in fake.calls if isinstance(c, int)) == [0, 1, 2] and fake.calls[0] == "begin"
    for p in net.parameters():
        assert torch.isfinite(p).all()


def test_timers_gather_through_a_transport_object():
    """With a transport set, the per-rank timer table is built by its small all-reduce (no torch.distributed call)."""
    from wallx_b200.utils.timers import Timers

    class _Comm:
        rank, world, device = 1, 4, "cpu"
        calls = 0

        def all_reduce_vector(self, t):
            _Comm.calls += 1
            out = t.clone()
            out[0] = 0.5  # what rank 0 contributed
            return out

    t = Timers(log_level=0)
    t("a", 0).start()
    t("a", 0).stop()
    t.set_comm(_Comm())
    table = t._get_elapsed_time_all_ranks(["a", "missing"], reset=False)
    assert table.shape == (4, 2) and _Comm.calls == 1
    assert table[1, 0] > 0 and table[0, 0] == 0.5 and float(table[:, 1].sum()) == 0.5  # row 0 is what the fake peer sent


def test_gather_flags_are_reset_when_the_number_of_copy_ctas_changes():
    """The ready flags of a gathered weight count the copy CTAs' arrivals per launch (target = copy CTAs x epoch), so a
    different number on the same weight must restart the count instead of meeting a target that is already, or never,
    reached."""
    from wallx_b200.parallel.zero3 import GatheredWeight

    flags = torch.full((3,), 40, dtype=torch.int32)
    g = GatheredWeight(512, 64, 2, 0, [0, 0], flags, torch.zeros(512, 64))
    g.epoch = 5
    g.pin_pullers(8)          # first launch fixes the number; earlier counts are this weight's own
    assert g.n_pullers == 8 and g.epoch == 5 and int(flags[0]) == 40
    g.pin_pullers(8)
    assert g.epoch == 5 and int(flags[0]) == 40
    g.pin_pullers(4)          # changed: flags and epoch start over
    assert g.n_pullers == 4 and g.epoch == 0 and int(flags.abs().sum()) == 0
    assert g.next_epoch() == 1

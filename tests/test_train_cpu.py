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


def _sharded_linear_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.distributed.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    from wallx_b200.parallel.ag_linear import AgLinear

    g = torch.Generator().manual_seed(0)
    full_w = torch.randn(8, 16, generator=g)
    bias = torch.randn(8, generator=g)
    lin = AgLinear(16, 8, None, "cpu", bias=True)
    lin.weight.load_full(full_w)
    with torch.no_grad():
        lin.bias.copy_(bias)
    assert lin.weight.shard.shape == (8 // world, 16)
    assert torch.equal(lin.weight.gather_full(), full_w)
    x = torch.randn(5, 16, generator=torch.Generator().manual_seed(10 + rank), requires_grad=True)
    y = lin(x)
    want = torch.nn.functional.linear(x.detach(), full_w, bias)
    assert torch.allclose(y, want, atol=1e-5)
    gy = torch.randn(5, 8, generator=torch.Generator().manual_seed(20 + rank))
    y.backward(gy)
    assert torch.allclose(x.grad, gy @ full_w, atol=1e-5)
    assert torch.allclose(lin.bias.grad, gy.sum(0), atol=1e-5)
    local_dw = gy.t() @ x.detach()
    shard_grad = lin.reduce_scatter_grad()
    torch.save({"local_dw": local_dw, "shard_grad": shard_grad}, os.path.join(tmp, f"agl_{rank}.pt"))
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world", [2, 4])
def test_sharded_weight_linear_over_gloo(tmp_path, world):
    """Shard arithmetic of the gathered-weight linear layer (rows per rank, gather, full-gradient accumulation,
    averaged reduce-scatter) with the collective stand-in that replaces the fused NVLink gather on CPU."""
    mp.spawn(_sharded_linear_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(tmp_path / f"agl_{r}.pt") for r in range(world)]
    mean_dw = sum(p["local_dw"] for p in parts) / world
    rows = 8 // world
    for r, p in enumerate(parts):
        assert torch.allclose(p["shard_grad"], mean_dw[r * rows:(r + 1) * rows], atol=1e-5)


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

    def reserve(self, total, dtype=torch.float32):
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

"""``QwenVlAct_Trainer``: the training loop behind ``train_qact.py``, driven by the reference's YAML.

Same constructor, same ``fit()`` and the same YAML keys as the reference trainer
(wall_x/trainer/qwen_vl_act_trainer.py:79-236, workspace/lerobot_example/config_qact.yml), but the
distributed machinery is this framework's own :class:`TrainEngine` (sharded optimizer state over a
hand-written NVLink transport) instead of accelerate + FSDP2, ranks come from ``torchrun``'s
environment, and the hot loop has no device synchronisation:

* the NaN/Inf policy is decided on the *reduced* gradient norm inside the optimizer kernel, so all
  ranks skip the same step (the reference's per-rank ``continue`` at :322-327 would hang FSDP);
* every logged scalar travels in one packed all-reduce per optimizer step (the reference issues ~75
  scalar gathers, :352-423);
* timers use CUDA events (no ``cuda.synchronize`` at every start).

Extra YAML keys (all optional): ``model`` (build from a preset instead of a checkpoint, for
synthetic runs), ``transport`` (``symm`` | ``dist``), ``optimizer_dtype``, ``log_interval``,
``max_steps``, ``step_save_interval``, ``step_timeout_s`` (host watchdog).
"""
from __future__ import annotations

import gc
import json
import os
import random
import time
from typing import Dict, Optional

import numpy as np
import torch

from ..config import tiny_config, wall_oss_config
from ..data.collator import to_device
from ..models import Qwen2_5_VLMoEForAction
from ..parallel.engine import TrainEngine
from ..utils.timers import Timers
from . import checkpoint as CK
from .logging import MetricLogger
from .schedule import CosineWithMinLR


def timer(func):
    """Wall-clock decorator for the slow set-up phases (reference: qwen_vl_act_trainer.py:29-50)."""
    import functools

    @functools.wraps(func)
    def wrapped(*a, **k):
        t0 = time.time()
        out = func(*a, **k)
        print_rank_last(f"[timer] {func.__name__}: {time.time() - t0:.2f}s")
        return out

    return wrapped


def _dist():
    return torch.distributed if (torch.distributed.is_available() and torch.distributed.is_initialized()) else None


def print_rank_last(msg: str) -> None:
    d = _dist()
    if d is None or d.get_rank() == d.get_world_size() - 1:
        print(msg, flush=True)


def seed_all(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


class StepWatchdog:
    """Host-side failure detector: a step that takes longer than ``timeout_s`` raises on the next
    check instead of letting the job sit forever on a dead peer."""

    def __init__(self, timeout_s: Optional[float]):
        self.timeout_s = timeout_s
        self.t0 = time.time()

    def kick(self):
        self.t0 = time.time()

    def check(self):
        if self.timeout_s and time.time() - self.t0 > self.timeout_s:
            raise TimeoutError(f"training step exceeded {self.timeout_s}s (peer failure or stall)")


class QwenVlAct_Trainer:
    @timer
    def __init__(self, config: Dict, logger=None, accelerator=None, seed: int = 42, data_config_path=None,
                 processor=None, dataset=None):
        for key in ("learning_rate", "num_epoch"):
            if key not in config:
                raise ValueError(f"config is missing required key '{key}'")
        from .config import TrainConfig

        self.typed_config = TrainConfig.from_dict(config).validate()  # wrong values fail here, by key name
        if self.typed_config.unknown_keys:
            print_rank_last(f"config: keys this trainer does not read: {self.typed_config.unknown_keys}")
        self.config = config
        self.logger = logger
        self.accelerator = accelerator  # accepted for signature compatibility; not used
        self.seed = seed
        d = _dist()
        self.world = d.get_world_size() if d else 1
        self.rank = d.get_rank() if d else 0
        self.is_main = self.rank == 0
        self.device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        seed_all(seed)
        self.epoch = 0
        self.global_step = 0
        self.initial_step = 0
        self.step_in_epoch = 0  # batches of the current epoch consumed at the last optimizer step
        self.grad_accum = int(config.get("gradient_accumulation_steps", 1))
        self.use_fast_tokenizer = bool(config.get("use_fast_tokenizer", False))
        self.processor = processor
        self._dataset = dataset
        self.metrics = MetricLogger(config.get("save_path"), config.get("log_project"), config.get("log_name"), config,
                                    use_wandb=bool(config.get("use_wandb", False)), is_main=self.is_main)
        from ..data.lerobot import get_data_configs

        self.data_config = get_data_configs(config.get("data", {}))
        self.load_model()
        if self.device.type == "cuda":
            print_rank_last(f"memory after model load: {torch.cuda.memory_allocated() / 2**30:.2f} GiB")
        self.load_qact_data()
        if "resume" in config and config["resume"]:
            self.resume_from_checkpoint()
        tok = self.model.processor.tokenizer if self.model.processor is not None else None
        self.action_token_id = tok.convert_tokens_to_ids("<|action|>") if tok is not None else None
        self.timers = Timers(log_level=0, log_option="minmax")
        if self.engine.transport == "symm":
            self.timers.set_comm(self.engine.symm)  # per-rank timer table over the own small all-reduce
        self.watchdog = StepWatchdog(config.get("step_timeout_s"))

    # ------------------------------------------------------------------ model / optimizer
    def _build_model(self) -> Qwen2_5_VLMoEForAction:
        cfg = self.config
        spec = cfg.get("model")
        if spec:  # synthetic / from-scratch model
            from ..data.synthetic import make_processor

            spec = dict(spec)
            preset = spec.pop("preset", "tiny")
            action_vocab = int(spec.pop("action_vocab", 16 if preset == "tiny" else 2048))
            overrides = dict(spec)
            for k in ("dof_config", "agent_pos_config"):
                if k in cfg and k not in overrides:
                    overrides[k] = cfg[k]
            mcfg = tiny_config(**overrides) if preset == "tiny" else wall_oss_config(action_vocab=action_vocab, **overrides)
            if self.processor is None:
                self.processor = make_processor(mcfg, action_vocab)
            return Qwen2_5_VLMoEForAction(mcfg, use_fast_tokenizer=self.use_fast_tokenizer, processor=self.processor)
        path = cfg["pretrained_wallx_path"]
        kw = {"processor": self.processor} if self.processor is not None else {}
        return Qwen2_5_VLMoEForAction.from_pretrained(
            path, use_fast_tokenizer=self.use_fast_tokenizer,
            action_tokenizer_path=cfg.get("action_tokenizer_path") if self.use_fast_tokenizer else None, **kw)

    def _param_group_fn(self):
        """(group, lr_scale, weight_decay) per parameter name -- the reference's three modes
        (qwen_vl_act_trainer.py:530-581): ``freeze_vlm``, ``action_expert_learning_rate``, plain."""
        cfg = self.config
        wd = float(cfg.get("weight_decay", 0.1))
        base_lr = float(cfg["learning_rate"])
        expert_lr = cfg.get("action_expert_learning_rate")

        def is_action(name: str) -> bool:
            return "moe.experts.1." in name or name.startswith("action_preprocessor.")

        if expert_lr is not None:
            scale = float(expert_lr) / base_lr
            return lambda name: ("action_expert", scale, wd) if is_action(name) else ("default", 1.0, wd)
        return lambda name: ("default", 1.0, wd)

    @timer
    def load_model(self):
        cfg = self.config
        model = self._build_model()
        if cfg.get("qwen_pretrain_path"):
            self.load_qwen_pretrain_weight(model, cfg["qwen_pretrain_path"])
        model = model.to(self.dtype).to(self.device)
        if cfg.get("freeze_vlm", False) or cfg.get("train_action_expert_only", False):
            for name, p in model.named_parameters():
                p.requires_grad_("moe.experts.1." in name or name.startswith("action_preprocessor."))
        self.model = model
        self.model_config = model.config
        self.processor = model.processor
        transport = cfg.get("transport", "symm" if self.device.type == "cuda" else "dist") if self.world > 1 else "local"
        symm = None
        if transport == "symm":
            from ..parallel.symm import SymmComm

            symm = SymmComm(torch.distributed.group.WORLD, self.device,
                            barrier_timeout_s=float(cfg.get("barrier_timeout_s", 30.0)))
        master = torch.float32
        if str(cfg.get("optimizer_dtype", "fp32")) in ("bf16", "bfloat16"):
            # the reference keeps bf16 Adam states; the fused CUDA update works on fp32 shards only (they are
            # sharded over the GPUs: 12 bytes per parameter divided by the world size). The CPU path honours bf16.
            if self.device.type == "cuda":
                raise ValueError("optimizer_dtype: bf16 is not available on CUDA: the fused AdamW kernel keeps fp32 "
                                 "master weights and moments; use optimizer_dtype: fp32")
            master = torch.bfloat16
        # parameter plan: `shard_params` (true = ZeRO-3 rows per rank, gather fused into the GEMMs; false = resident
        # bf16 parameters). Unset, it follows the reference's `FSDP2` key (train_qact.py:42-49), default off.
        shard = cfg.get("shard_params")
        if shard is None:
            shard = bool(cfg.get("FSDP2", False)) and self.world > 1
        self.engine = TrainEngine(model, lr=float(cfg["learning_rate"]), weight_decay=float(cfg.get("weight_decay", 0.1)),
                                  max_grad_norm=float(cfg.get("max_grad_norm", 1.0)), grad_accum=self.grad_accum,
                                  world=self.world, rank=self.rank, transport=transport, symm=symm,
                                  param_group_fn=self._param_group_fn(), master_dtype=master, shard_params=bool(shard))
        self.status_check_interval = int(cfg.get("status_check_interval", 1))
        # per-unit reduce-scatter during backward (own transport only; YAML key `overlap_reduce`, default on)
        self.engine.overlap_reduce = transport == "symm" and bool(cfg.get("overlap_reduce", True))
        self.lr_scheduler = CosineWithMinLR(float(cfg["learning_rate"]), int(cfg.get("num_warmup_steps", 0)),
                                            int(cfg.get("num_training_steps", 1_000_000)), float(cfg.get("min_lr", 0.0)))
        model.enable_input_require_grads()

    @timer
    def load_qwen_pretrain_weight(self, model, path: str):
        """Initialise from a stock Qwen2.5-VL checkpoint: its dense MLP becomes expert 0."""
        state = CK.rename_qwen_to_moe(CK.load_safetensors_dir(path))
        missing, unexpected = model.load_state_dict(state, strict=False)
        print_rank_last(f"qwen pretrain load: {len(missing)} missing, {len(unexpected)} unexpected keys")

    @timer
    def load_qact_data(self):
        cfg = self.config
        from ..data import lerobot as LR

        if self._dataset is not None:
            base = self._dataset
        elif cfg.get("data", {}).get("use_lerobot", False) and not cfg.get("data", {}).get("synthetic", False):
            pre = LR.load_lerobot_data(cfg, cfg["data"]["lerobot_config"], rank=self.rank, world_size=self.world,
                                       seed=self.seed, processor=self.processor, model_config=self.model_config)
            self.dataset = pre
            return
        else:
            sc = cfg.get("data", {}).get("synthetic_config", {})
            A = sum(self.model_config.dof_config.values())
            base = LR.SyntheticEpisodeDataset(n=int(sc.get("num_samples", 64)), image_hw=tuple(sc.get("image_hw", (96, 128))),
                                              action_dim=min(A, 20), horizon=self.data_config["action_horizon"] - 1,
                                              seed=self.seed)
        self.dataset = LR.PreprocessedDataset(base, cfg, self.data_config, seed=self.seed, rank=self.rank,
                                              world_size=self.world, processor=self.processor,
                                              model_config=self.model_config)
        d = _dist()
        if d:
            d.barrier()

    # ------------------------------------------------------------------ loops
    def fit(self):
        cfg = self.config
        if cfg.get("resume", {}) and cfg["resume"].get("validate_first", False):
            self.val_loop()
        for epoch in range(self.epoch, int(cfg["num_epoch"])):
            self.epoch = epoch
            self.train_loop(epoch)
            if (epoch + 1) % int(cfg.get("epoch_save_interval", 10)) == 0:
                self.save_checkpoint(epoch)
            self.val_loop()
            gc.collect()
            if cfg.get("max_steps") and self.global_step >= int(cfg["max_steps"]):
                break
        self.metrics.close()

    def _fit_action_dims(self, batch):
        """The collator pads actions to 20 dims; a model with fewer DOFs takes the leading ones."""
        A = self.model.action_preprocessor.action_dim
        P = self.model.action_preprocessor.propri_dim
        for k, w in (("action_chunk", A), ("dof_mask", A), ("proprioception", P), ("agent_pos_mask", P)):
            if k in batch and batch[k].shape[-1] != w:
                batch[k] = batch[k][..., :w]
        return batch

    def _reduce_metrics(self, vals: Dict[str, torch.Tensor]) -> Dict[str, float]:
        """One packed all-reduce for every scalar of the step, then a single host read."""
        keys = sorted(vals.keys())
        t = torch.stack([vals[k].detach().float().reshape(()) for k in keys]).to(self.device)
        d = _dist()
        if d and self.world > 1:
            symm = getattr(self.engine, "symm", None) if getattr(self, "engine", None) is not None else None
            if symm is not None and self.engine.transport == "symm":
                t = symm.all_reduce_vector(t)  # own small all-reduce over NVLink: no NCCL call on the step path
            else:
                d.all_reduce(t)
        return dict(zip(keys, t.cpu().tolist()))

    def train_loop(self, epoch: int):
        cfg = self.config
        model, engine = self.model, self.engine
        model.train()
        loader, sampler = self.dataset.get_train_dataloader()
        sampler.set_epoch(epoch)
        prof = self._profiler()
        log_every = int(cfg.get("log_interval", 1))
        acc: Dict[str, torch.Tensor] = {}
        t_iter = time.time()
        self.timers("interval-time", 0).start()
        n_batches = len(loader) if hasattr(loader, "__len__") else None
        skip = self.initial_step  # resuming inside an epoch: the first `skip` batches were already trained on
        for i, batch in enumerate(loader):
            if i < skip:
                continue
            self.watchdog.check()
            self.timers("data-load", 0).start()
            batch = to_device(self._fit_action_dims(batch), self.device, self.dtype)
            self.timers("data-load", 0).stop()
            self.timers("forward-compute", 0).start()
            out = model(mode="train", **batch)
            self.timers("forward-compute", 0).stop()
            self.timers("backward-compute", 0).start()
            # the optimizer step follows this micro-batch: at every accumulation boundary and at the end of the loader
            steps_now = (i + 1) % self.grad_accum == 0 or (n_batches is not None and i + 1 == n_batches)
            engine.backward(out.loss, last=steps_now)
            self.timers("backward-compute", 0).stop()

            def add(name, v):
                if v is not None:
                    acc[name] = acc.get(name, 0) + v.detach().float() / self.grad_accum
            add("train_loss", out.loss)
            add("cross_entropy_loss", out.cross_entropy_loss)
            add("flow_loss", out.flow_loss)
            if out.channel_loss_dict:
                for k, v in out.channel_loss_dict.items():
                    if k == "action_accuracy":
                        add("action_accuracy", v)
                    elif out.channel_loss_count_dict and k in out.channel_loss_count_dict:
                        acc[f"_sum_{k}"] = acc.get(f"_sum_{k}", 0) + v.detach().float()
                        acc[f"_cnt_{k}"] = acc.get(f"_cnt_{k}", 0) + out.channel_loss_count_dict[k].detach().float()
            if steps_now:
                # (a remainder at the end of the loader is stepped on with the gradient averaged over the
                # micro-batches actually accumulated, as accelerate does for the reference at the end of its dataloader)
                self.timers("optimizer", 0).start()
                lr = self.lr_scheduler.get_lr()
                n_micro = engine._micro
                engine.optimizer_step(lr)
                self.lr_scheduler.step()
                self.global_step += 1
                self.step_in_epoch = i + 1
                self.timers("optimizer", 0).stop()
                self.watchdog.kick()
                if n_micro != self.grad_accum:
                    acc = {k: (v * (self.grad_accum / max(n_micro, 1)) if not k.startswith("_") else v) for k, v in acc.items()}
                if self.status_check_interval and self.global_step % self.status_check_interval == 0:
                    engine.check_status()  # raises on every rank alike when some rank's device-side wait ran out
                if self.global_step % log_every == 0:
                    acc["total_norm"] = engine.grad_norm() * self.world  # averaged below
                    red = self._reduce_metrics(acc)
                    logd = {"lr": lr}
                    for k, v in red.items():
                        if k.startswith("_sum_"):
                            name = k[5:]
                            cnt = red.get(f"_cnt_{name}", 0.0)
                            if cnt > 0:
                                logd[f"channel_loss_{name}"] = v / cnt
                        elif not k.startswith("_cnt_"):
                            logd[k] = v / self.world
                    self.metrics.log(logd, step=self.global_step)
                    self.training_log(epoch, i, logd, time.time() - t_iter)
                    t_iter = time.time()
                acc = {}
                if cfg.get("step_save_interval") and self.global_step % int(cfg["step_save_interval"]) == 0:
                    self.save_checkpoint(epoch, self.global_step)
                if cfg.get("max_steps") and self.global_step >= int(cfg["max_steps"]):
                    break
            if prof is not None:
                prof.step()
        self.timers("interval-time", 0).stop()
        if prof is not None:
            prof.__exit__(None, None, None)
        self.initial_step = 0
        self.step_in_epoch = 0

    def _profiler(self):
        cfg = self.config
        if not cfg.get("profile", False):
            return None
        from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler

        prof = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA],
                       schedule=schedule(wait=int(cfg.get("profile_wait_iters", 10)),
                                         warmup=int(cfg.get("profile_warmup_iters", 5)),
                                         active=int(cfg.get("profile_active_iters", 2))),
                       on_trace_ready=tensorboard_trace_handler(cfg.get("profile_save_path", "./profile"),
                                                                worker_name=f"worker{self.rank}"),
                       record_shapes=True, profile_memory=True, with_stack=True)
        prof.__enter__()
        return prof

    @torch.no_grad()
    def val_loop(self):
        model = self.model
        model.eval()
        loader, _ = self.dataset.get_val_dataloader()
        total = torch.zeros((), device=self.device)
        count = torch.zeros((), device=self.device)
        for batch in loader:
            batch = to_device(self._fit_action_dims(batch), self.device, self.dtype)
            out = model(mode="validate", return_logits=False, **batch)
            if out.loss is not None:
                total += out.loss.detach().float()
                count += 1
        red = self._reduce_metrics({"s": total, "c": count})
        val = red["s"] / max(red["c"], 1.0)
        self.metrics.log({"val_loss": val}, step=self.global_step)
        print_rank_last(f"[val] epoch {self.epoch} step {self.global_step} val_loss {val:.5f}")
        model.train()
        return val

    def print_rank0(self, msg, flush: bool = True) -> None:
        """Print on the main rank only."""
        if self.is_main:
            print(msg, flush=flush)

    def _load_fsdp_state_dict_with_distribute_tensor(self, ckpt_path: str) -> None:
        """Reference name of the sharded resume path (qwen_vl_act_trainer.py:797-837: full safetensors file ->
        ``distribute_tensor`` per parameter). Here parameters are resident on every rank, so the file is loaded
        as is and each rank refreshes its fp32 master shard from it."""
        state = CK.strip_prefixes(CK.load_safetensors_dir(ckpt_path))
        with self.engine.gathered_parameters(writeback=True):
            self.model.load_state_dict(state, strict=False)

    def training_log(self, epoch, iteration, logd, seconds):
        msg = (f"epoch {epoch} iter {iteration} step {self.global_step} loss {logd.get('train_loss', float('nan')):.5f} "
               f"lr {logd['lr']:.3e} grad_norm {logd.get('total_norm', float('nan')):.3f} time {seconds:.3f}s")
        print_rank_last(msg)
        self.timers.log(["interval-time", "data-load", "forward-compute", "backward-compute", "optimizer"], reset=True)

    def log_l1_details(self, pred, gt, dof_mask, step=None):
        """Per-DOF-group L1 between predicted and ground-truth actions (``detail/l1_loss_<dof>``)."""
        out = {}
        l1 = (pred.float() - gt.float()).abs() * dof_mask.float()
        out["base_l1_loss"] = float(l1.sum() / dof_mask.float().sum().clamp_min(1))
        start = 0
        for name, width in self.model_config.dof_config.items():
            seg = l1[..., start:start + width]
            msk = dof_mask[..., start:start + width].float()
            if msk.sum() > 0:
                out[f"detail/l1_loss_{name}"] = float(seg.sum() / msk.sum())
            start += width
        self.metrics.log(out, step=step if step is not None else self.global_step)
        return out

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, epoch: int, step: int = 0):
        """``<save_path>/<epoch>[_<step>]/``: consolidated HF weights (rank 0) + one optimizer shard
        file per rank + a manifest that allows resuming on a different world size."""
        root = self.config.get("save_path")
        if not root:
            return None
        name = f"{epoch}_{step}" if step else f"{epoch}"
        path = os.path.join(root, name)
        os.makedirs(path, exist_ok=True)
        with self.engine.gathered_parameters():  # collective when parameters are row-sharded
            if self.is_main:
                self.model.save_pretrained(path)
        if self.is_main:
            with open(os.path.join(path, "trainer_state.json"), "w", encoding="utf-8") as f:
                json.dump({"epoch": epoch, "global_step": self.global_step, "world": self.world,
                           "step_in_epoch": self.step_in_epoch if step else 0, "mid_epoch": bool(step),
                           "scheduler": self.lr_scheduler.state_dict(), "seed": self.seed}, f)
        state = self.engine.optimizer_state()
        state["rng"] = {"torch": torch.get_rng_state(), "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None}
        torch.save(state, os.path.join(path, f"optim_rank{self.rank:05d}_of_{self.world:05d}.pt"))
        d = _dist()
        if d:
            d.barrier()
        return path

    def resume_from_checkpoint(self):
        r = self.config["resume"]
        path = r["ckpt"]
        state = CK.strip_prefixes(CK.load_safetensors_dir(path))
        # the loaded bf16 weights replace the owners' shards and refresh the fp32 masters on exit
        with self.engine.gathered_parameters(writeback=True):
            missing, unexpected = self.model.load_state_dict(state, strict=False)
        print_rank_last(f"resume: loaded weights from {path} ({len(missing)} missing, {len(unexpected)} unexpected)")
        if r.get("load_ckpt_only", False):
            return
        ts = os.path.join(path, "trainer_state.json")
        if os.path.exists(ts):
            with open(ts, "r", encoding="utf-8") as f:
                st = json.load(f)
            if st.get("mid_epoch"):  # a step checkpoint: continue the same epoch after the batches already seen
                self.epoch = int(st["epoch"])
                self.initial_step = self.step_in_epoch = int(st.get("step_in_epoch", 0))
            else:
                self.epoch = int(st["epoch"]) + 1
            self.global_step = int(st["global_step"])
            self.lr_scheduler.load_state_dict(st["scheduler"])
            from ..parallel.reshard import load_optimizer_shards

            load_optimizer_shards(self.engine, path, int(st["world"]))

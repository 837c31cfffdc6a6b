"""Typed view of the training YAML with validation.

The trainer keeps reading the plain dict, exactly like the reference (train_qact.py:22-30 loads the YAML into a
dict and qwen_vl_act_trainer.py reads it with ``config[...]`` / ``.get``; only ``learning_rate`` and ``num_epoch``
are checked there, :125-128). This module adds what that lacks: every known key has a type, a default and a range,
a wrong value fails at start-up with the key's name instead of somewhere inside the first step, and unknown
top-level keys are reported (not rejected: user configs carry extra bookkeeping keys).
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional

_TRANSPORTS = ("auto", "symm", "dist", "local")
_OPT_DTYPES = ("fp32", "float32", "bf16", "bfloat16")


@dataclass
class ResumeConfig:
    ckpt: Optional[str] = None
    load_ckpt_only: bool = False
    validate_first: bool = False


@dataclass
class TrainConfig:
    # required by the reference too
    learning_rate: float = 0.0
    num_epoch: int = 0
    # what to train
    model_type: str = "qwen2_5"
    pretrained_wallx_path: Optional[str] = None
    qwen_pretrain_path: Optional[str] = None       # stock Qwen2.5-VL weights mapped onto expert 0
    model: Optional[Dict[str, Any]] = None         # overrides of config.json (tests and synthetic runs)
    save_path: Optional[str] = None
    use_fast_tokenizer: bool = False
    action_tokenizer_path: Optional[str] = None
    log_project: Optional[str] = None
    log_name: Optional[str] = None
    use_wandb: bool = False
    # optimisation
    min_lr: float = 0.0
    num_warmup_steps: int = 0
    num_training_steps: int = 0
    batch_size_per_gpu: int = 8
    eval_batch_size_per_gpu: Optional[int] = None
    gradient_accumulation_steps: int = 1
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    epoch_save_interval: int = 1
    step_save_interval: Optional[int] = None
    log_interval: int = 1
    max_steps: Optional[int] = None
    padding_side: str = "left"
    num_workers: int = 4
    freeze_vlm: bool = False
    train_action_expert_only: bool = False
    action_expert_learning_rate: Optional[float] = None
    # engine
    FSDP2: bool = True
    torch_compile: bool = False
    transport: str = "auto"
    overlap_reduce: bool = True
    optimizer_dtype: str = "fp32"
    shard_params: Optional[bool] = None  # ZeRO-3 rows per rank; unset = follow FSDP2 on more than one GPU
    barrier_timeout_s: float = 30.0      # bound of every device-side wait on a peer (own transport)
    status_check_interval: int = 1       # optimizer steps between host reads of the device status words (0 = never)
    step_timeout_s: Optional[float] = None
    # profiler window
    profile: bool = False
    profile_save_path: Optional[str] = None
    profile_wait_iters: int = 10
    profile_warmup_iters: int = 5
    profile_active_iters: int = 2
    # nested sections, kept as given
    dof_config: Dict[str, int] = field(default_factory=dict)
    agent_pos_config: Dict[str, int] = field(default_factory=dict)
    data: Dict[str, Any] = field(default_factory=dict)
    resume: Optional[ResumeConfig] = None
    unknown_keys: List[str] = field(default_factory=list)

    @classmethod
    def from_dict(cls, config: Dict[str, Any]) -> "TrainConfig":
        known = {f.name for f in fields(cls)} - {"unknown_keys"}
        kw: Dict[str, Any] = {}
        kinds = {f.name: str(f.type) for f in fields(cls)}
        for k, v in config.items():
            if k in known and v is not None:
                if isinstance(v, str):  # YAML 1.1 reads `9e-5` as a string; the trainer applies float() / int() itself
                    try:
                        if "float" in kinds[k]:
                            v = float(v)
                        elif "int" in kinds[k] and "Dict" not in kinds[k]:
                            v = int(v)
                    except ValueError:
                        pass
                kw[k] = v
        r = config.get("resume")
        if isinstance(r, dict) and r:
            extra = set(r) - {"ckpt", "load_ckpt_only", "validate_first"}
            if extra:
                raise ValueError(f"config key 'resume' has unknown entries {sorted(extra)}")
            kw["resume"] = ResumeConfig(**r)
        else:
            kw.pop("resume", None)
        out = cls(**kw)
        out.unknown_keys = sorted(k for k in config if k not in known)
        return out

    def validate(self, require_paths: bool = False) -> "TrainConfig":
        def fail(key: str, why: str):
            raise ValueError(f"config key '{key}': {why} (got {getattr(self, key)!r})")

        for key in ("learning_rate", "min_lr", "weight_decay", "max_grad_norm"):
            v = getattr(self, key)
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                fail(key, "must be a number")
            if v < 0:
                fail(key, "must not be negative")
        if self.learning_rate <= 0:
            fail("learning_rate", "must be positive")
        if self.min_lr > self.learning_rate:
            fail("min_lr", "must not exceed learning_rate")
        if self.action_expert_learning_rate is not None and not (isinstance(self.action_expert_learning_rate, (int, float))
                                                                 and self.action_expert_learning_rate > 0):
            fail("action_expert_learning_rate", "must be a positive number")
        for key, low in (("num_epoch", 1), ("batch_size_per_gpu", 1), ("gradient_accumulation_steps", 1), ("epoch_save_interval", 1),
                         ("num_warmup_steps", 0), ("num_training_steps", 0), ("num_workers", 0), ("profile_wait_iters", 0),
                         ("profile_warmup_iters", 0), ("profile_active_iters", 1)):
            v = getattr(self, key)
            if isinstance(v, bool) or not isinstance(v, int):
                fail(key, "must be an integer")
            if v < low:
                fail(key, f"must be at least {low}")
        for key in ("step_save_interval", "max_steps"):
            v = getattr(self, key)
            if v is not None and (isinstance(v, bool) or not isinstance(v, int) or v < 1):
                fail(key, "must be a positive integer")
        if isinstance(self.log_interval, bool) or not isinstance(self.log_interval, int) or self.log_interval < 1:
            fail("log_interval", "must be a positive integer")
        if self.eval_batch_size_per_gpu is not None and (not isinstance(self.eval_batch_size_per_gpu, int) or self.eval_batch_size_per_gpu < 1):
            fail("eval_batch_size_per_gpu", "must be a positive integer")
        for key in ("use_fast_tokenizer", "FSDP2", "torch_compile", "overlap_reduce", "profile", "freeze_vlm", "train_action_expert_only",
                    "use_wandb"):
            if not isinstance(getattr(self, key), bool):
                fail(key, "must be true or false")
        if self.shard_params is not None and not isinstance(self.shard_params, bool):
            fail("shard_params", "must be true or false")
        if not (isinstance(self.barrier_timeout_s, (int, float)) and 0 < self.barrier_timeout_s <= 600):
            fail("barrier_timeout_s", "must be a number of seconds in (0, 600]")
        if isinstance(self.status_check_interval, bool) or not isinstance(self.status_check_interval, int) or self.status_check_interval < 0:
            fail("status_check_interval", "must be a non-negative integer")
        if self.transport not in _TRANSPORTS:
            fail("transport", f"must be one of {_TRANSPORTS}")
        if str(self.optimizer_dtype) not in _OPT_DTYPES:
            fail("optimizer_dtype", f"must be one of {_OPT_DTYPES}")
        if self.padding_side not in ("left", "right"):
            fail("padding_side", "must be 'left' or 'right'")
        if self.step_timeout_s is not None and not (isinstance(self.step_timeout_s, (int, float)) and self.step_timeout_s > 0):
            fail("step_timeout_s", "must be a positive number of seconds")
        for key in ("dof_config", "agent_pos_config"):
            table = getattr(self, key)
            if not isinstance(table, dict) or any(not isinstance(n, int) or isinstance(n, bool) or n < 1 for n in table.values()):
                fail(key, "must map each key to a positive integer width")
        if self.dof_config and sum(self.dof_config.values()) > 20:
            fail("dof_config", "widths add up to more than the 20 padded action dimensions")
        if self.agent_pos_config and sum(self.agent_pos_config.values()) > 20:
            fail("agent_pos_config", "widths add up to more than the 20 padded proprioception dimensions")
        if not isinstance(self.data, dict):
            fail("data", "must be a mapping")
        if self.profile and not self.profile_save_path:
            fail("profile_save_path", "is needed when profile is true")
        if self.resume is not None and not self.resume.ckpt:
            raise ValueError("config key 'resume': 'ckpt' (checkpoint directory) is missing")
        if require_paths:
            for key in ("pretrained_wallx_path", "save_path"):
                if not getattr(self, key):
                    fail(key, "must be set")
        return self

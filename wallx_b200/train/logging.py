"""Metric sinks: stdout + JSONL always, Weights & Biases when it is installed and asked for.

Metric names are the reference's (``lr, train_loss, cross_entropy_loss, flow_loss,
channel_loss_<dataset>, action_accuracy, total_norm, val_loss``; qwen_vl_act_trainer.py:355-433).
"""
from __future__ import annotations

import json
import os
import time
from typing import Dict, Optional


class MetricLogger:
    def __init__(self, directory: Optional[str] = None, project: Optional[str] = None, name: Optional[str] = None,
                 config: Optional[Dict] = None, use_wandb: bool = False, is_main: bool = True):
        self.is_main = is_main
        self.file = None
        self.wandb = None
        if not is_main:
            return
        if directory:
            os.makedirs(directory, exist_ok=True)
            self.file = open(os.path.join(directory, "metrics.jsonl"), "a", encoding="utf-8")
        if use_wandb:
            try:
                import wandb

                self.wandb = wandb
                wandb.init(project=project, name=name, config=config or {})
            except Exception as e:  # wandb is optional and absent on this image
                print(f"wandb not available ({e}); logging to stdout/JSONL only")

    def log(self, metrics: Dict[str, float], step: Optional[int] = None) -> None:
        if not self.is_main:
            return
        rec = {"step": step, "time": time.time(), **{k: (float(v) if hasattr(v, "__float__") else v) for k, v in metrics.items()}}
        if self.file:
            self.file.write(json.dumps(rec) + "\n")
            self.file.flush()
        if self.wandb is not None:
            self.wandb.log(metrics, step=step)

    def close(self):
        if self.file:
            self.file.close()

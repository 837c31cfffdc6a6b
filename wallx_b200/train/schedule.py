"""Learning-rate schedule: linear warm-up then cosine decay to a floor.

Same curve as the HF ``get_cosine_with_min_lr_schedule_with_warmup`` the reference builds at
qwen_vl_act_trainer.py:583-592 (``min_lr`` absolute, half a cosine period by default).
"""
from __future__ import annotations

import math


class CosineWithMinLR:
    def __init__(self, base_lr: float, num_warmup_steps: int, num_training_steps: int, min_lr: float = 0.0,
                 num_cycles: float = 0.5):
        self.base_lr = float(base_lr)
        self.warmup = int(num_warmup_steps)
        self.total = int(num_training_steps)
        self.min_ratio = float(min_lr) / float(base_lr) if base_lr > 0 else 0.0
        self.num_cycles = num_cycles
        self.step_count = 0

    def factor(self, step: int) -> float:
        if step < self.warmup:
            return float(step) / float(max(1, self.warmup))
        progress = float(step - self.warmup) / float(max(1, self.total - self.warmup))
        f = 0.5 * (1.0 + math.cos(math.pi * self.num_cycles * 2.0 * progress))
        f = f * (1 - self.min_ratio) + self.min_ratio
        return max(0.0, f)

    def get_lr(self) -> float:
        return self.base_lr * self.factor(self.step_count)

    def get_last_lr(self):
        return [self.get_lr()]

    def step(self) -> None:
        self.step_count += 1

    def state_dict(self):
        return {"step_count": self.step_count, "base_lr": self.base_lr, "warmup": self.warmup, "total": self.total,
                "min_ratio": self.min_ratio, "num_cycles": self.num_cycles}

    def load_state_dict(self, sd):
        self.step_count = int(sd["step_count"])

"""Fused, sharded AdamW over flat buffers.

One kernel per (buffer, hyper-parameter segment) does: gradient scale (1 / accumulation steps and
the global-norm clip coefficient, read from a device scalar -- no host sync), decoupled weight
decay, Adam moments, fp32 master update and the bf16 parameter write. A non-finite global norm
skips the update on every rank alike (the reference's per-rank ``isnan -> continue``,
qwen_vl_act_trainer.py:322-327, would desynchronise ranks).

Semantics of ``torch.optim.AdamW`` + ``clip_grad_norm_`` as configured by the reference
(qwen_vl_act_trainer.py:335-337, 530-581): weight decay on every parameter, default betas / eps.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from ..ops import _ext
from ..ops import ref
from ..parallel.flat import FlatBuffer


class FlatAdamW:
    def __init__(self, buffers: Sequence[FlatBuffer], lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, max_grad_norm: float = 1.0, grad_accum: int = 1):
        self.buffers = list(buffers)
        self.lr = lr
        self.betas = betas
        self.eps = eps
        self.weight_decay = weight_decay
        self.max_grad_norm = max_grad_norm
        self.grad_accum = grad_accum
        self.step_count = 0
        dev = self.buffers[0].device
        self.norm_sq = torch.zeros(1, device=dev, dtype=torch.float32)
        self._hyper_cache = {}

    # -------------------------------------------------------------- norm
    def local_grad_sumsq(self, shard_only: bool = False) -> torch.Tensor:
        """Sum of squared gradient elements (device scalar). With ``shard_only`` only this rank's
        shard of every buffer is counted (after a reduce-scatter the shards partition the model)."""
        self.norm_sq.zero_()
        for b in self.buffers:
            g = b.grad[b.shard_range[0]:b.shard_range[1]] if shard_only else b.grad
            if g.is_cuda:
                _ext.get().sumsq_bf16(g, self.norm_sq)
            else:
                self.norm_sq += (g.float() ** 2).sum()
        return self.norm_sq

    # -------------------------------------------------------------- step
    def _hyper(self, dev, lr, wd):
        b1, b2 = self.betas
        t = self.step_count
        vals = [lr, b1, b2, self.eps, wd, 1 - b1 ** t, 1 - b2 ** t, self.max_grad_norm or -1.0, 1.0 / self.grad_accum]
        return torch.tensor(vals, dtype=torch.float32).to(dev, non_blocking=True)

    def step(self, lr: Optional[float] = None, norm_sq: Optional[torch.Tensor] = None,
             grad_shards: Optional[List[torch.Tensor]] = None) -> None:
        """Update every buffer's shard. ``norm_sq`` is the (already all-reduced) squared global norm
        of the unscaled gradients; ``grad_shards[i]`` overrides the gradient source of buffer i (the
        reduce-scattered shard)."""
        self.step_count += 1
        lr = self.lr if lr is None else lr
        for i, b in enumerate(self.buffers):
            s0, s1 = b.shard_range
            g_all = grad_shards[i] if grad_shards is not None else b.grad[s0:s1]
            p16 = b.param[s0:s1]
            for lo, hi, seg in b.update_ranges():
                wd = seg.weight_decay
                seg_lr = lr * seg.lr_scale
                if b.param.is_cuda:
                    hyper = self._hyper(b.device, seg_lr, wd)
                    fn = _ext.get().adamw_step_f32g if g_all.dtype == torch.float32 else _ext.get().adamw_step
                    fn(p16[lo:hi], b.master[lo:hi], b.exp_avg[lo:hi], b.exp_avg_sq[lo:hi], g_all[lo:hi], hyper, norm_sq)
                else:
                    self._cpu_step(b, lo, hi, g_all, seg_lr, wd, norm_sq)

    def _cpu_step(self, b, lo, hi, g_all, lr, wd, norm_sq):
        scale = 1.0 / self.grad_accum
        if norm_sq is not None:
            n2 = float(norm_sq.item())
            if not math.isfinite(n2):
                return
            if self.max_grad_norm and self.max_grad_norm > 0:
                coef = self.max_grad_norm / (math.sqrt(n2) * scale + 1e-6)
                if coef < 1.0:
                    scale *= coef
        ref.adamw_step(b.master[lo:hi], g_all[lo:hi], b.exp_avg[lo:hi], b.exp_avg_sq[lo:hi], self.step_count, lr,
                       self.betas[0], self.betas[1], self.eps, wd, scale)
        s0 = b.shard_range[0]
        b.param[s0 + lo:s0 + hi].copy_(b.master[lo:hi].to(b.param.dtype))

    def zero_grad(self) -> None:
        for b in self.buffers:
            b.zero_grad()
            b.clear_touched()

    def state_dict(self):
        return {"step": self.step_count, "buffers": [b.state_dict() for b in self.buffers]}

    def load_state_dict(self, sd):
        self.step_count = int(sd["step"])
        for b, s in zip(self.buffers, sd["buffers"]):
            b.master.copy_(s["master"])
            b.exp_avg.copy_(s["exp_avg"])
            b.exp_avg_sq.copy_(s["exp_avg_sq"])

"""Optional NVTX ranges around the fused operator paths.

With ``WALLX_NVTX=1`` in the environment every public operator of ``wallx_b200.ops.functional`` (and the engine's
optimizer step) pushes a named NVTX range, so a timeline shows ``linear``, ``moe_ffn``, ``attention_packed``,
``lm_head_ce`` ... instead of bare kernel names. Without the variable nothing is wrapped and the call path is
unchanged (the reference has NVTX hooks in its timers only, wall_x/utils/timers.py:160-171, never enabled).
"""
from __future__ import annotations

import functools
import os
from typing import Iterable


def enabled() -> bool:
    return os.environ.get("WALLX_NVTX", "0") not in ("", "0", "false", "False")


def wrap(fn, name: str):
    import torch

    @functools.wraps(fn)
    def ranged(*args, **kwargs):
        if not torch.cuda.is_available():
            return fn(*args, **kwargs)
        torch.cuda.nvtx.range_push(name)
        try:
            return fn(*args, **kwargs)
        finally:
            torch.cuda.nvtx.range_pop()

    ranged.__wrapped_by_nvtx__ = True
    return ranged


def annotate_module(module, names: Iterable[str], prefix: str = "wx.") -> int:
    """Replace ``module.<name>`` by a ranged version for every listed function; returns how many were wrapped."""
    if not enabled():
        return 0
    n = 0
    for name in names:
        fn = getattr(module, name, None)
        if callable(fn) and not getattr(fn, "__wrapped_by_nvtx__", False):
            setattr(module, name, wrap(fn, prefix + name))
            n += 1
    return n

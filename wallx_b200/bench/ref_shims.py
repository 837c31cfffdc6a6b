"""Compatibility shims that let the *unmodified* reference package (installed under
``baseline/_ref``) import and run on this image.

The reference pins torch 2.6 / transformers 4.49 and needs peft, torchdiffeq and qwen_vl_utils;
the image has torch 2.11 / transformers 5.5 and none of those three. Nothing in the reference's own
files is touched: missing third-party modules are provided as tiny stand-ins in ``sys.modules`` and
symbols that transformers 5 removed or changed are added back to the transformers namespaces
before the reference is imported.
"""
from __future__ import annotations

import sys
import types


def _stub(name: str, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    return m


def install(ref_dir: str) -> None:
    import torch
    import torch.nn as nn

    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    for k in [k for k in sys.modules if k == "wall_x" or k.startswith("wall_x.")]:
        del sys.modules[k]  # never mix with the alias package of the same name

    # ---- third-party packages absent from the image
    if "peft" not in sys.modules:
        _stub("peft", LoraConfig=lambda **k: k, get_peft_model=lambda m, c: m)
    if "torchdiffeq" not in sys.modules:
        def odeint(func, y0, t, method="euler", **kw):
            assert method == "euler"
            ys, y = [y0], y0
            for i in range(len(t) - 1):
                y = y + (t[i + 1] - t[i]) * func(t[i], y)
                ys.append(y)
            return torch.stack(ys)

        _stub("torchdiffeq", odeint=odeint)
    if "qwen_vl_utils" not in sys.modules:
        q = _stub("qwen_vl_utils")
        q.vision_process = _stub("qwen_vl_utils.vision_process", MIN_PIXELS=4 * 28 * 28, MAX_PIXELS=16384 * 28 * 28,
                                 IMAGE_FACTOR=28)

    # ---- transformers 4.49 names that 5.x dropped
    import transformers.cache_utils as cu

    if not hasattr(cu, "SlidingWindowCache"):
        cu.SlidingWindowCache = type("SlidingWindowCache", (cu.StaticCache,), {})
    import transformers.models.qwen2_vl.modeling_qwen2_vl as q2

    if not hasattr(q2, "Qwen2RMSNorm"):
        class Qwen2RMSNorm(nn.Module):
            def __init__(self, hidden_size, eps=1e-6):
                super().__init__()
                self.weight = nn.Parameter(torch.ones(hidden_size))
                self.variance_epsilon = eps

            def forward(self, hidden_states):
                dt = hidden_states.dtype
                h = hidden_states.to(torch.float32)
                h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + self.variance_epsilon)
                return self.weight * h.to(dt)

        q2.Qwen2RMSNorm = Qwen2RMSNorm
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS

    if "default" not in ROPE_INIT_FUNCTIONS:
        def _default_rope(config, device=None, seq_len=None, **kw):
            base = config.rope_theta
            dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
            inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.int64).to(device=device, dtype=torch.float) / dim))
            return inv, 1.0

        ROPE_INIT_FUNCTIONS["default"] = _default_rope

    # ---- transformers 5 builds its own (nested-config) Qwen2.5-VL inside the base class constructor;
    # the reference replaces every one of those sub-modules right after, and its flat config has no
    # ``text_config``. Keep only the PreTrainedModel part of that constructor.
    import transformers.models.qwen2_5_vl.modeling_qwen2_5_vl as m25

    if not getattr(m25.Qwen2_5_VLForConditionalGeneration, "_wallx_ref_shim", False):
        def _base_init(self, config, *a, **k):
            m25.Qwen2_5_VLPreTrainedModel.__init__(self, config)

        m25.Qwen2_5_VLForConditionalGeneration.__init__ = _base_init
        m25.Qwen2_5_VLForConditionalGeneration._wallx_ref_shim = True

    # ---- transformers 5 re-initialises rotary buffers through a method that 4.49-era rotary classes
    # do not have; such modules already computed their buffers in their own constructor.
    import transformers.modeling_utils as mu

    if not getattr(mu.PreTrainedModel, "_wallx_ref_shim", False):
        _orig_init_weights = mu.PreTrainedModel._init_weights

        def _init_weights(self, module):
            if "RotaryEmbedding" in module.__class__.__name__ and not hasattr(module, "compute_default_rope_parameters"):
                return
            return _orig_init_weights(self, module)

        mu.PreTrainedModel._init_weights = _init_weights
        mu.PreTrainedModel._wallx_ref_shim = True

    # ---- transformers 5 renamed the class flag ``_supports_flash_attn_2`` to ``_supports_flash_attn``
    if not getattr(mu.PreTrainedModel, "_wallx_ref_fa_shim", False):
        _orig_can = mu.PreTrainedModel._flash_attn_can_dispatch

        def _can_dispatch(self, *a, **k):
            if getattr(self, "_supports_flash_attn_2", False) and not getattr(self, "_supports_flash_attn", False):
                type(self)._supports_flash_attn = True
            return _orig_can(self, *a, **k)

        mu.PreTrainedModel._flash_attn_can_dispatch = _can_dispatch
        mu.PreTrainedModel._wallx_ref_fa_shim = True

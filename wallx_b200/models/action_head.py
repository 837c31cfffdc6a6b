"""Action head: per-robot normaliser, flow-matching noise schedule, action/proprio embedders.

Numerical conventions follow the reference's ``wall_x/model/action_head.py``:
``x_t = (1 - t) * eps + t * a``, target ``a - eps`` (:336-338); ``t = (s - u) / s`` with
``u ~ Beta(alpha, beta)`` per sample (:253-271); time enters as a raw [0, 1] scalar through a
sinusoidal embedding ``cat(sin, cos)`` (:129-163); embedding MLP ``w3(silu(w2(cat[w1(cat[x_t,
mask]), sin(t)])))`` (:343-360); flow loss = elementwise MSE * dof_mask, unreduced (:401-425).
Unlike the reference (:232-233) nothing here is pinned to a CUDA device.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn

from ..utils.constant import action_statistic_dof
from .layers import Linear


class Normalizer(nn.Module):
    """Per-robot min/delta tables as non-trainable ``ParameterDict``s (checkpoint-compatible)."""

    def __init__(self, statistics: Dict, dof_config: Dict[str, int]):
        super().__init__()
        mins, deltas = {}, {}
        for robot, stats in statistics.items():
            mn, dl = [], []
            for key, width in dof_config.items():
                if key in stats:
                    mn.extend(stats[key]["min"])
                    dl.extend(stats[key]["delta"])
                else:
                    mn.extend([0.0] * width)
                    dl.extend([1.0] * width)
            mins[robot] = nn.Parameter(torch.tensor(mn, dtype=torch.float32), requires_grad=False)
            deltas[robot] = nn.Parameter(torch.tensor(dl, dtype=torch.float32), requires_grad=False)
        self.min = nn.ParameterDict(mins)
        self.delta = nn.ParameterDict(deltas)

    @staticmethod
    def _names(dataset_names: Sequence[str]) -> List[str]:
        return [n for n in dataset_names if n != "x2_multimodal"]

    def normalize_data(self, xs, dataset_names):
        out = []
        for x, name in zip(xs, self._names(dataset_names)):
            mn, dl = self.min[name].to(x.device, x.dtype), self.delta[name].to(x.device, x.dtype)
            out.append(torch.clamp((x - mn) / dl * 2 - 1, -1, 1))
        return torch.stack(out)

    def unnormalize_data(self, xs, dataset_names, dof_mask=None):
        out = []
        masks = dof_mask if dof_mask is not None else [None] * len(xs)
        for x, name, mask in zip(xs, self._names(dataset_names), masks):
            mn, dl = self.min[name].to(x.device, x.dtype), self.delta[name].to(x.device, x.dtype)
            if mask is not None:
                sel = mask[0].bool()
                mn, dl = mn[sel], dl[sel]
            out.append((x + 1) / 2 * dl + mn)
        return torch.stack(out)


class SinusoidalPosEmb(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.dim = dim

    def forward(self, t: torch.Tensor) -> torch.Tensor:
        half = self.dim // 2
        k = math.log(10000) / (half - 1)
        freq = torch.exp(torch.arange(half, device=t.device, dtype=torch.float32) * -k)
        ang = t.float()[:, None] * freq[None, :]
        return torch.cat((ang.sin(), ang.cos()), dim=-1)


class ActionProcessor(nn.Module):
    def __init__(self, config, verbose: bool = False):
        super().__init__()
        self.dof_config = config.dof_config
        self.agent_pos_config = config.agent_pos_config
        self.action_dim = sum(self.dof_config.values())
        self.propri_dim = sum(self.agent_pos_config.values())
        self.hidden_size = config.hidden_size
        if verbose:
            print(f"ActionProcessor: action_dim={self.action_dim} propri_dim={self.propri_dim}", flush=True)
        self.normalizer_action = Normalizer(action_statistic_dof, config.dof_config)
        self.normalizer_propri = Normalizer(action_statistic_dof, config.agent_pos_config)
        ns = config.noise_scheduler or {}
        self.beta_alpha = float(ns.get("beta_alpha", 1.5))
        self.beta_beta = float(ns.get("beta_beta", 1.0))
        self.s = float(ns.get("s", 0.999))
        self.time_embed = SinusoidalPosEmb(config.hidden_size)
        self.propri_proj = Linear(self.propri_dim * 2, self.hidden_size, bias=False)
        self.w1 = Linear(self.action_dim * 2, self.hidden_size, bias=False)
        self.w2 = Linear(self.hidden_size * 2, self.hidden_size, bias=False)
        self.w3 = Linear(self.hidden_size, self.hidden_size, bias=False)
        self.action_proj_back = Linear(self.hidden_size, self.action_dim, bias=False)

    # ------------------------------------------------------------------ sampling
    def sample_time(self, batch_size: int, device, dtype, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """t = (s - u) / s, u ~ Beta(alpha, beta). Sampled as a ratio of Gammas on the host RNG when a
        generator is given (reproducible), else through torch.distributions on ``device``."""
        if generator is not None:
            a = torch._standard_gamma(torch.full((batch_size,), self.beta_alpha), generator=generator)
            b = torch._standard_gamma(torch.full((batch_size,), self.beta_beta), generator=generator)
            u = (a / (a + b)).to(device=device, dtype=dtype)
        else:
            dist = torch.distributions.Beta(torch.tensor(self.beta_alpha, device=device),
                                            torch.tensor(self.beta_beta, device=device))
            u = dist.sample([batch_size]).to(dtype)
        return (self.s - u) / self.s

    # ------------------------------------------------------------------ embedders
    def proprioception_proj(self, proprioception, dataset_names=None, dof_mask=None, use_history=False):
        w = self.propri_proj.weight
        x = proprioception.to(device=w.device, dtype=w.dtype)
        if dof_mask is not None:
            x = torch.cat([x, dof_mask.to(device=w.device, dtype=w.dtype)], dim=-1)
        return self.propri_proj(x)

    def _embed(self, noisy_action, time, dof_mask):
        w_dtype = self.w1.weight.dtype
        if dof_mask is not None:
            noisy_action = torch.cat([noisy_action, dof_mask.to(noisy_action.dtype)], dim=-1)
        a = self.w1(noisy_action.to(w_dtype))
        te = self.time_embed(time).to(w_dtype).unsqueeze(1).expand(-1, a.shape[1], -1)
        h = self.w2(torch.cat([a, te], dim=-1))
        return self.w3(torch.nn.functional.silu(h))

    def forward(self, action_chunk, dataset_names=None, dof_mask=None, noise=None, time=None, generator=None):
        """Returns ``(action_embeddings [B, L, H], flow_target [B, L, A])`` for flow-matching training."""
        B = action_chunk.shape[0]
        if noise is None:
            if generator is not None:
                noise = torch.randn(action_chunk.shape, generator=generator).to(action_chunk.device, action_chunk.dtype)
            else:
                noise = torch.randn_like(action_chunk)
        if time is None:
            time = self.sample_time(B, action_chunk.device, action_chunk.dtype, generator)
        t = time.view(B, 1, 1).to(action_chunk.dtype)
        noisy = (1 - t) * noise + t * action_chunk
        flow = action_chunk - noise
        return self._embed(noisy, time, dof_mask), flow

    def step(self, timestep, noisy_action, dof_mask=None):
        """Embedding of the current noisy actions at ``timestep [B]`` (inference)."""
        return self._embed(noisy_action, timestep, dof_mask)

    def flow_loss(self, action_hidden_states, flow, dof_mask=None):
        pred = self.action_proj_back(action_hidden_states)
        loss = (pred.float() - flow.float()) ** 2
        if dof_mask is not None:
            loss = loss * dof_mask.reshape(-1, dof_mask.shape[-1]).float()
        return loss

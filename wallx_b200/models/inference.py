"""Inference paths: flow-matching action sampling with a reused prefix KV cache, and
autoregressive text / FAST generation.

Reference behaviour (modeling_qwen2_5_vl_act.py:1538-1981): ``predict_mode="diffusion"`` draws
``x0 ~ N(0, I)`` and integrates ``dx/dt = v(x, t)`` from 0 to 1 with explicit Euler on
``linspace(0, 1, n)``, re-running the *whole* sequence through the LLM at every evaluation;
``"text"`` / ``"fast"`` split the prompt at ``<|im_start|>assistant`` and run HF ``generate``.

Here the prefix (every token before the first ``<|action|>``) goes through the model once and its
keys/values are kept per layer; each Euler evaluation then runs only the suffix tokens (the action
chunk) against the cached prefix. This is exact: under both attention rules the prefix never sees
the action tokens. ``num_inference_timesteps`` counts Euler *evaluations* here (10 by default);
pass ``reference_grid=True`` to reproduce the reference's ``linspace(0, 1, n)`` grid with ``n - 1``
evaluations. The Euler loop can be captured in a CUDA graph (``use_cuda_graph=True``).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..ops import functional as F_
from ..ops.gemm import inference_kernels
from .llm import KVCache, StepContext


def _ids_of(model, name, default):
    tok = getattr(getattr(model, "processor", None), "tokenizer", None)
    if tok is None:
        return default
    try:
        v = tok.convert_tokens_to_ids(name)
        return default if v is None else v
    except Exception:
        return default


class FlowSampler:
    """Prefix pass + Euler steps for one batch. Build once per observation, call :meth:`sample`."""

    def __init__(self, model, input_ids, attention_mask=None, position_ids=None, moe_token_types=None,
                 pixel_values=None, pixel_values_videos=None, image_grid_thw=None, video_grid_thw=None,
                 proprioception=None, agent_pos_mask=None, dataset_names=None, dof_mask=None, second_per_grid_ts=None,
                 image_grid_host=None, video_grid_host=None, pack_index=None, seq_lens=None, **_unused):
        from .vla import PackInfo

        self.model = model
        cfg = model.config
        dev = model.device
        B, S = input_ids.shape
        input_ids = input_ids.to(dev)
        if attention_mask is not None:
            attention_mask = attention_mask.to(dev)
        action_id = model.action_token_id_set["action_token_id"]
        if moe_token_types is None:
            moe_token_types = (input_ids == action_id).long()
        pos, _ = model._positions(input_ids, position_ids.to(dev) if position_ids is not None else None, attention_mask,
                                  image_grid_thw, video_grid_thw, second_per_grid_ts)
        pack = PackInfo.build(attention_mask, B, S, dev, seq_lens, pack_index)
        self.pack = pack
        ids = input_ids.reshape(-1).index_select(0, pack.pack_index)
        types = moe_token_types.to(dev).reshape(-1).index_select(0, pack.pack_index).to(torch.int32)
        pos3 = pos.reshape(3, -1).index_select(1, pack.pack_index)
        emb = model._embed_packed(ids, pack, pixel_values, image_grid_thw, pixel_values_videos, video_grid_thw,
                                  proprioception, agent_pos_mask, dataset_names, image_grid_host, video_grid_host)

        # ---- split every sequence at its first action token (host side; ids are small)
        ids_host = ids.cpu().tolist()
        self.B = B
        pre_rows, suf_rows, pre_lens, suf_lens = [], [], [], []
        for b in range(B):
            s0, s1 = pack.cu[b], pack.cu[b + 1]
            seq = ids_host[s0:s1]
            first = seq.index(action_id) if action_id in seq else len(seq)
            assert first < len(seq), "No action token found in input_ids"
            pre_rows.extend(range(s0, s0 + first))
            suf_rows.extend(range(s0 + first, s1))
            pre_lens.append(first)
            suf_lens.append(len(seq) - first)
        self.pre_lens, self.suf_lens = pre_lens, suf_lens
        pre_idx = torch.tensor(pre_rows, device=dev, dtype=torch.long)
        suf_idx = torch.tensor(suf_rows, device=dev, dtype=torch.long)
        self.suf_ids = ids.index_select(0, suf_idx)
        self.suf_is_action = self.suf_ids == action_id
        self.n_action = int(sum(1 for r in suf_rows if ids_host[r] == action_id))
        self.horizon = self.n_action // B
        self.pre_idx, self.suf_idx = pre_idx, suf_idx
        self.suf_emb_static = None
        hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        caps = [p + s for p, s in zip(pre_lens, suf_lens)]
        self.cache = KVCache(cfg.num_hidden_layers, caps, hkv * d, dev, emb.dtype)
        bidir_on = cfg.action_attn == "bidirectional"

        # ---- prefix pass: fills the cache (keys/values after rotary), hidden states are not needed
        cu_pre = [0]
        for l in pre_lens:
            cu_pre.append(cu_pre[-1] + l)
        pre_cache_rows = torch.cat([self.cache.slot_rows(b, 0, pre_lens[b]) for b in range(B)]) if pre_rows else \
            torch.zeros(0, dtype=torch.long, device=dev)
        pre_types = types.index_select(0, pre_idx)
        meta_pre = F_.AttnMeta(cu_pre, dev, causal=True, cache_rows=pre_cache_rows,
                               k_starts=[self.cache.offsets[b] for b in range(B)], k_lens=pre_lens,
                               k_rows=self.cache.offsets[-1])
        cos, sin = model.model.rotary(pos3.index_select(1, pre_idx))
        plan = F_.make_route_plan(pre_types, cfg.num_experts) if cfg.mlp_moe else None
        F_.RoutePlan.note_single_expert(plan, pre_types)
        meta_pre.device_tables(dev)
        self.ctx_pre = StepContext(meta_pre, cos, sin, plan, cache=self.cache, cache_mode="prefill")

        # ---- per-step context over the suffix tokens
        cu_suf = [0]
        for l in suf_lens:
            cu_suf.append(cu_suf[-1] + l)
        suf_cache_rows = torch.cat([self.cache.slot_rows(b, pre_lens[b], suf_lens[b]) for b in range(B)])
        suf_types = types.index_select(0, suf_idx)
        bq = (suf_types == 1) if bidir_on else None
        bk = None
        if bidir_on:
            bk = torch.zeros(self.cache.offsets[-1], dtype=torch.bool, device=dev)
            bk[suf_cache_rows] = suf_types == 1
        meta_suf = F_.AttnMeta(cu_suf, dev, causal=True, bidir_q=bq, bidir_k=bk, cache_rows=suf_cache_rows,
                               k_starts=[self.cache.offsets[b] for b in range(B)], k_lens=caps,
                               k_rows=self.cache.offsets[-1])
        meta_suf.device_tables(dev)
        cos_s, sin_s = model.model.rotary(pos3.index_select(1, suf_idx))
        plan_s = F_.make_route_plan(suf_types, cfg.num_experts) if cfg.mlp_moe else None
        F_.RoutePlan.note_single_expert(plan_s, suf_types)
        self.ctx = StepContext(meta_suf, cos_s, sin_s, plan_s, cache=self.cache, cache_mode="step")
        self.dof_mask = dof_mask.to(dev, emb.dtype) if dof_mask is not None else None
        self.action_rows = torch.nonzero(self.suf_is_action, as_tuple=False).squeeze(1)
        self.dtype = emb.dtype
        self.device = dev
        self._graph = None
        self.prefill(emb)

    def prefill(self, emb: torch.Tensor) -> None:
        """Run the prefix tokens of packed embeddings ``emb [T, H]`` through the model (fills the KV
        cache) and keep the suffix rows (action placeholders and what follows them). Shapes and
        buffer addresses do not change between calls, so this can be replayed from a CUDA graph."""
        x = emb.index_select(0, self.pre_idx)
        if x.shape[0] > 0:
            for layer in self.model.model.layers:
                x = layer(x, self.ctx_pre)
        suf = emb.index_select(0, self.suf_idx)
        if self.suf_emb_static is None:
            self.suf_emb_static = suf
        else:
            self.suf_emb_static.copy_(suf)

    # ------------------------------------------------------------------
    def velocity(self, t: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """v(x, t) for ``x [B, horizon, A]`` and a scalar time tensor ``t`` (device)."""
        m = self.model
        B, L, A = x.shape
        a_emb = m.action_preprocessor.step(t.reshape(1).expand(B), x, self.dof_mask).reshape(B * L, -1)
        if self.suf_emb_static.shape[0] == B * L:
            h = a_emb
        else:
            h = self.suf_emb_static.index_copy(0, self.action_rows, a_emb)
        for layer in m.model.layers:
            h = layer(h, self.ctx)
        h = m.model.norm(h)
        if h.shape[0] != B * L:
            h = h.index_select(0, self.action_rows)
        return m.action_preprocessor.action_proj_back(h).reshape(B, L, A)

    def sample(self, x0: torch.Tensor, num_steps: int = 10, reference_grid: bool = False,
               use_cuda_graph: bool = False) -> torch.Tensor:
        """Explicit Euler from t=0 to t=1. ``num_steps`` evaluations of the velocity field
        (``reference_grid``: the reference's ``linspace(0, 1, num_steps)`` -> ``num_steps - 1``)."""
        n_eval = num_steps - 1 if reference_grid else num_steps
        times = torch.linspace(0, 1, n_eval + 1, device=self.device, dtype=torch.float32)
        x = x0.to(self.device, self.dtype)
        if use_cuda_graph and x.is_cuda:
            return self._sample_graph(x, times, n_eval)
        for i in range(n_eval):
            dt = (times[i + 1] - times[i]).to(self.dtype)
            x = x + dt * self.velocity(times[i].to(self.dtype), x)
        return x

    def _sample_graph(self, x, times, n_eval):
        key = (tuple(x.shape), n_eval)
        if self._graph is None or self._graph[0] != key:
            static_x = x.clone()
            times_d = times.to(self.dtype)

            def loop(xx):
                for i in range(n_eval):
                    xx = xx + (times_d[i + 1] - times_d[i]) * self.velocity(times_d[i], xx)
                return xx

            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                loop(static_x)  # warm-up outside capture (allocator, attribute set-up)
            torch.cuda.current_stream().wait_stream(s)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                static_out = loop(static_x)
            self._graph = (key, g, static_x, static_out)
        _, g, static_x, static_out = self._graph
        static_x.copy_(x)
        g.replay()
        return static_out.clone()


@inference_kernels()
@torch.no_grad()
def predict_flow(model, pred_horizon=None, action_dim=None, input_ids=None, action_chunk=None, dataset_names=None,
                 dof_mask=None, num_inference_timesteps=10, noise=None, reference_grid=False, use_cuda_graph=False,
                 **batch) -> Dict[str, torch.Tensor]:
    sampler = FlowSampler(model, input_ids, dataset_names=dataset_names, dof_mask=dof_mask, **batch)
    B = input_ids.shape[0]
    horizon = pred_horizon if pred_horizon is not None else sampler.horizon
    A = action_dim if action_dim is not None else model.action_preprocessor.action_dim
    if noise is None:
        noise = torch.randn((B, horizon, A), device=sampler.device, dtype=sampler.dtype)
    x = sampler.sample(noise, num_inference_timesteps, reference_grid, use_cuda_graph)
    names = list(dataset_names) if dataset_names is not None else ["x2_normal"] * B
    out = {"predict_action": model.action_preprocessor.normalizer_action.unnormalize_data(x.float(), names)}
    if action_chunk is not None:
        out["gt_action"] = model.action_preprocessor.normalizer_action.unnormalize_data(
            action_chunk.to(sampler.device).float(), names)
    return out


def _pdl_switch(on: bool):
    """Turn programmatic dependent launch of the small inference kernels on (when the extension is there) and return
    the setter, so that the caller can turn it off again."""
    from ..ops import _ext

    C = _ext.get(required=False)
    if C is None or not hasattr(C, "set_pdl"):
        return lambda _on: None
    C.set_pdl(bool(on))
    return C.set_pdl


class FlowEngine:
    """Serving engine for a fixed observation layout: one CUDA graph per action chunk.

    A robot controller sends the same prompt template at every step: the positions of the image,
    proprioception and action placeholders, the image sizes and the batch size do not change, only
    the pixel values, the proprioception, the text ids and the noise do. The engine analyses that
    layout once (host side), keeps static device buffers for the inputs, and captures the whole
    chunk -- embedding, ViT, prefix pass that fills the KV cache, ``num_steps`` Euler evaluations
    reusing it, un-normalisation -- in one CUDA graph. A call copies the new inputs into the static
    buffers, replays the graph and returns the chunk; no Python runs per kernel and nothing is
    allocated. Reference behaviour being replaced: modeling_qwen2_5_vl_act.py:1886-1981.
    """

    INPUT_KEYS = ("input_ids", "pixel_values", "proprioception", "agent_pos_mask", "dof_mask")

    def __init__(self, model, example: Dict, num_inference_timesteps: int = 10, reference_grid: bool = False,
                 use_cuda_graph: bool = True):
        self.model = model
        dev = model.device
        fdtype = model.model.embed_tokens.weight.dtype
        self.steps, self.reference_grid = num_inference_timesteps, reference_grid
        self.static: Dict[str, torch.Tensor] = {}
        for k in self.INPUT_KEYS:
            v = example.get(k)
            if torch.is_tensor(v):
                self.static[k] = v.to(dev, fdtype if v.is_floating_point() else v.dtype).clone()
        self.names = list(example.get("dataset_names") or ["x2_normal"] * example["input_ids"].shape[0])
        self.grid = example.get("image_grid_thw")
        self.grid_host = example.get("image_grid_host")
        if self.grid_host is None and self.grid is not None:
            self.grid_host = [[int(v) for v in g] for g in self.grid.tolist()]
        layout = {k: v for k, v in example.items() if k not in self.INPUT_KEYS and k not in ("action_chunk", "labels")}
        layout["image_grid_host"] = self.grid_host
        with torch.no_grad(), inference_kernels():
            self.sampler = FlowSampler(model, self.static["input_ids"], dataset_names=self.names,
                                       pixel_values=self.static.get("pixel_values"),
                                       proprioception=self.static.get("proprioception"),
                                       agent_pos_mask=self.static.get("agent_pos_mask"),
                                       dof_mask=self.static.get("dof_mask"),
                                       **{k: v for k, v in layout.items() if k != "dataset_names"})
        self.sampler.dof_mask = self.static.get("dof_mask")  # the sampler reads the static buffer
        B = example["input_ids"].shape[0]
        A = model.action_preprocessor.action_dim
        self.noise = torch.zeros(B, self.sampler.horizon, A, device=dev, dtype=fdtype)
        cfg = model.config
        ids_host = example["input_ids"].cpu()
        specials = [cfg.image_token_id, cfg.video_token_id, model.action_token_id_set["action_token_id"],
                    model.action_token_id_set["propri_token_id"]]
        self._special_ids = specials
        self._signature = self._layout_signature(ids_host)
        self.out = None
        self.graph = None
        with torch.no_grad():
            self._run()  # eager warm-up: builds every cached table before capture
            if use_cuda_graph and dev.type == "cuda":
                # Inside the graph the small kernels of the denoise loop are launched as programmatic dependents:
                # each one's prologue overlaps the tail of the kernel before it (csrc/launch.h).
                pdl = _pdl_switch(os.environ.get("WALLX_PDL", "1") == "1")
                try:
                    torch.cuda.synchronize(dev)
                    side = torch.cuda.Stream(device=dev)
                    side.wait_stream(torch.cuda.current_stream(dev))
                    with torch.cuda.stream(side):
                        self._run()
                    torch.cuda.current_stream(dev).wait_stream(side)
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        self._run()
                    self.graph = g
                finally:
                    pdl(False)

    def _layout_signature(self, ids_host: torch.Tensor) -> torch.Tensor:
        sig = torch.zeros_like(ids_host, dtype=torch.int8)
        for i, t in enumerate(self._special_ids):
            sig[ids_host == t] = i + 1
        return sig

    @inference_kernels()
    def _run(self) -> None:
        s, m = self.sampler, self.model
        ids = self.static["input_ids"].reshape(-1).index_select(0, s.pack.pack_index)
        emb = m._embed_packed(ids, s.pack, self.static.get("pixel_values"), self.grid, None, None,
                              self.static.get("proprioception"), self.static.get("agent_pos_mask"), self.names,
                              self.grid_host, None)
        s.prefill(emb)
        x = s.sample(self.noise, self.steps, self.reference_grid, use_cuda_graph=False)
        self.out = m.action_preprocessor.normalizer_action.unnormalize_data(x.float(), self.names)

    @torch.no_grad()
    def __call__(self, batch: Optional[Dict] = None, noise: Optional[torch.Tensor] = None, check_layout: bool = True,
                 **kw) -> Dict[str, torch.Tensor]:
        batch = dict(batch or {}, **kw)
        ids = batch.get("input_ids")
        if check_layout and torch.is_tensor(ids) and ids.device.type == "cpu":
            if ids.shape != self._signature.shape or not torch.equal(self._layout_signature(ids), self._signature):
                raise ValueError("FlowEngine: the observation layout changed (placeholder positions or shape); "
                                 "build a new engine for it")
        for k, buf in self.static.items():
            v = batch.get(k)
            if torch.is_tensor(v):
                buf.copy_(v, non_blocking=True)
        if noise is not None:
            self.noise.copy_(noise, non_blocking=True)
        else:
            self.noise.normal_()
        if self.graph is not None:
            self.graph.replay()
        else:
            self._run()
        return {"predict_action": self.out.clone()}


# ------------------------------------------------------------------------------------ text / FAST
class _Decoder:
    """Prefill + one-token-at-a-time decoding for a batch of prompts with per-sample KV slots."""

    def __init__(self, model, max_new_tokens: int, input_ids, attention_mask=None, moe_token_types=None, **mm):
        from .vla import PackInfo

        self.model = model
        cfg = model.config
        dev = model.device
        B, S = input_ids.shape
        input_ids = input_ids.to(dev)
        if attention_mask is not None:
            attention_mask = attention_mask.to(dev)
        pos, deltas = model._positions(input_ids, None, attention_mask, mm.get("image_grid_thw"), mm.get("video_grid_thw"),
                                       mm.get("second_per_grid_ts"))
        pack = PackInfo.build(attention_mask, B, S, dev, mm.get("seq_lens"), mm.get("pack_index"))
        ids = input_ids.reshape(-1).index_select(0, pack.pack_index)
        pos3 = pos.reshape(3, -1).index_select(1, pack.pack_index)
        types = torch.zeros_like(ids, dtype=torch.int32)
        emb = model._embed_packed(ids, pack, mm.get("pixel_values"), mm.get("image_grid_thw"),
                                  mm.get("pixel_values_videos"), mm.get("video_grid_thw"), mm.get("proprioception"),
                                  mm.get("agent_pos_mask"), mm.get("dataset_names"), mm.get("image_grid_host"),
                                  mm.get("video_grid_host"))
        hkv, d = cfg.num_key_value_heads, cfg.head_dim
        self.B, self.dev = B, dev
        self.lens = list(pack.seq_lens)
        caps = [l + max_new_tokens for l in self.lens]
        self.cache = KVCache(cfg.num_hidden_layers, caps, hkv * d, dev, emb.dtype)
        # next rope position per sample = max position so far + 1
        self.next_pos = torch.stack([pos3[:, pack.cu[b]:pack.cu[b + 1]].max() + 1 for b in range(B)]).to(torch.long)
        rows = torch.cat([self.cache.slot_rows(b, 0, self.lens[b]) for b in range(B)])
        meta = F_.AttnMeta(pack.cu, dev, causal=True, cache_rows=rows,
                           k_starts=[self.cache.offsets[b] for b in range(B)], k_lens=self.lens,
                           k_rows=self.cache.offsets[-1])
        cos, sin = model.model.rotary(pos3)
        plan = F_.make_route_plan(types, cfg.num_experts) if cfg.mlp_moe else None
        if plan is not None:
            plan.single_expert = 0  # text generation: every token goes through the VLM expert
        ctx = StepContext(meta, cos, sin, plan, cache=self.cache, cache_mode="prefill")
        h = model.model(emb, ctx)
        last = torch.tensor([c - 1 for c in pack.cu[1:]], device=dev)
        self.last_hidden = h.index_select(0, last)

    def logits(self) -> torch.Tensor:
        return F_.linear(self.last_hidden, self.model.lm_head.weight).float()

    def step(self, tokens: torch.Tensor) -> None:
        """Append one token per sample and compute the hidden state at it."""
        m, cfg, B, dev = self.model, self.model.config, self.B, self.dev
        emb = m.model.embed_tokens(tokens)
        rows = torch.cat([self.cache.slot_rows(b, self.lens[b], 1) for b in range(B)])
        self.lens = [l + 1 for l in self.lens]
        meta = F_.AttnMeta(list(range(B + 1)), dev, causal=True, cache_rows=rows,
                           k_starts=[self.cache.offsets[b] for b in range(B)], k_lens=self.lens,
                           k_rows=self.cache.offsets[-1])
        pos3 = self.next_pos.view(1, B).expand(3, B)
        self.next_pos = self.next_pos + 1
        cos, sin = m.model.rotary(pos3)
        plan = F_.make_route_plan(torch.zeros(B, dtype=torch.int32, device=dev), cfg.num_experts) if cfg.mlp_moe else None
        if plan is not None:
            plan.single_expert = 0
        ctx = StepContext(meta, cos, sin, plan, cache=self.cache, cache_mode="step")
        self.last_hidden = m.model(emb, ctx)


@inference_kernels()
@torch.no_grad()
def generate(model, input_ids, max_new_tokens: int = 100, do_sample: bool = False, temperature: float = 1.0,
             eos_token_id=None, pad_token_id=None, top_k: Optional[int] = None, generator=None, **mm) -> torch.Tensor:
    """Greedy or temperature sampling; returns ``[B, S + new]`` ids (prompt included, as HF does)."""
    eos = set(eos_token_id if isinstance(eos_token_id, (list, tuple)) else ([eos_token_id] if eos_token_id is not None else []))
    pad = pad_token_id if pad_token_id is not None else (next(iter(eos)) if eos else 0)
    dec = _Decoder(model, max_new_tokens, input_ids, **mm)
    B = input_ids.shape[0]
    done = torch.zeros(B, dtype=torch.bool, device=dec.dev)
    new_tokens: List[torch.Tensor] = []
    for i in range(max_new_tokens):
        logits = dec.logits()
        if do_sample:
            logits = logits / max(temperature, 1e-5)
            if top_k:
                kth = logits.topk(top_k, dim=-1).values[:, -1:]
                logits = logits.masked_fill(logits < kth, float("-inf"))
            probs = torch.softmax(logits, dim=-1)
            nxt = torch.multinomial(probs, 1, generator=generator).squeeze(1)
        else:
            nxt = logits.argmax(-1)
        nxt = torch.where(done, torch.full_like(nxt, pad), nxt)
        new_tokens.append(nxt)
        if eos:
            for e in eos:
                done = done | (nxt == e)
            if bool(done.all()):
                break
        if i + 1 < max_new_tokens:
            dec.step(nxt)
    gen = torch.stack(new_tokens, dim=1) if new_tokens else input_ids.new_zeros((B, 0))
    return torch.cat([input_ids.to(dec.dev), gen], dim=1)


@inference_kernels()
@torch.no_grad()
def predict_text(model, predict_mode: str, pred_horizon=None, action_dim=None, input_ids=None, attention_mask=None,
                 pixel_values=None, image_grid_thw=None, action_chunk=None, proprioception=None, dataset_names=None,
                 dof_mask=None, agent_pos_mask=None, re_generate=False, labels=None, image_grid_host=None,
                 max_new_tokens: int = 100) -> Dict[str, object]:
    out: Dict[str, object] = {}
    im_start = _ids_of(model, "<|im_start|>", 151644)
    assistant = _ids_of(model, "assistant", 77091)
    row = input_ids[0]
    match = (row[:-1] == im_start) & (row[1:] == assistant)
    if not bool(match.any()):
        raise ValueError("input_ids does not contain the generation prompt tokens <|im_start|>assistant")
    split = int(torch.nonzero(match)[0].item())
    gt_ids = input_ids[:, split + 3:]
    prompt = input_ids[:, : split + 3]
    am = attention_mask[:, : split + 3] if attention_mask is not None else None
    proc = model.processor
    out["input_text"] = proc.batch_decode(prompt, skip_special_tokens=False, clean_up_tokenization_spaces=True)
    tok = proc.tokenizer
    pred_ids = generate(model, prompt, max_new_tokens=max_new_tokens, do_sample=bool(re_generate),
                        temperature=0.7 if re_generate else 1.0, eos_token_id=[tok.eos_token_id],
                        pad_token_id=tok.pad_token_id, attention_mask=am, pixel_values=pixel_values,
                        image_grid_thw=image_grid_thw, proprioception=proprioception, agent_pos_mask=agent_pos_mask,
                        dataset_names=dataset_names, image_grid_host=image_grid_host)
    out["gt_output_text"] = proc.batch_decode(gt_ids, skip_special_tokens=False, clean_up_tokenization_spaces=True)
    out["predict_output_text"] = proc.batch_decode(pred_ids, skip_special_tokens=False, clean_up_tokenization_spaces=True)
    if predict_mode == "fast":
        start = tok.init_kwargs["action_token_start_index"]
        action_id = [int(t) - start for t in pred_ids[0].tolist() if int(t) >= start]
        decoder = getattr(proc, "action_processor", None)
        if decoder is None:
            raise RuntimeError("predict_mode='fast' needs processor.action_processor (the FAST tokenizer) to decode ids")
        import numpy as np

        pa = decoder.decode([action_id], time_horizon=pred_horizon, action_dim=action_dim)
        if np.sum(pa) == 0:
            out["predict_action"] = None
        else:
            pa = torch.tensor(pa, device=model.device)
            dm = dof_mask.to(model.device) if dof_mask is not None else None
            out["predict_action"] = model.action_preprocessor.normalizer_action.unnormalize_data(pa, dataset_names, dm)
        if action_chunk is not None and dof_mask is not None:
            ac = action_chunk[:, :, dof_mask[0, 0, :].bool()]
            out["gt_action"] = model.action_preprocessor.normalizer_action.unnormalize_data(
                ac.to(model.device), dataset_names, dof_mask.to(model.device))
        else:
            out["gt_action"] = None
    return out

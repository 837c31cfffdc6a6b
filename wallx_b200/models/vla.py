"""``Qwen2_5_VLMoEForAction``: vision tower + dual-expert LLM + action head, with the reference's
public surface (``from_pretrained``, ``forward(mode=...)``, ``predict``, ``predict_action``,
``generate``; modeling_qwen2_5_vl_act.py:735-2336) on top of the packed-token B200 operator layer.

What is kept: argument names, batch keys, output fields, loss definitions, state-dict key layout.
What is different by design:
* sequences are packed (padding rows never enter a kernel);
* the LM head runs only on rows that carry a label (training) and logits are materialised for all
  positions only when asked for (``return_logits=True``, default outside ``mode="train"``);
* flow-matching inference fills a prefix KV cache once and runs the Euler steps over the action
  tokens only (the reference re-runs the whole sequence each step, :1906-1952);
* no host synchronisation is needed when the batch carries the host-side packing info that
  :func:`wallx_b200.data.collator.add_pack_info` attaches (``pack_index``, ``seq_lens``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, List, Optional

import torch
import torch.nn as nn

from ..config import Qwen2_5_VLConfig
from ..ops import functional as F_
from ..ops import index as IX
from .action_head import ActionProcessor
from .layers import Linear
from .generation import GenerationHooksMixin
from .llm import Qwen2_5_VLMoEModel, StepContext
from .vision import VisionTransformer

ACTION_DATASET_NAMES: List[str] = []
MULTIMODAL_DATASET_NAMES: List[str] = []


def _dataset_names():
    global ACTION_DATASET_NAMES, MULTIMODAL_DATASET_NAMES
    if not ACTION_DATASET_NAMES:
        from ..data.config import ACTION_DATASET_NAMES as A, MULTIMODAL_DATASET_NAMES as M

        ACTION_DATASET_NAMES, MULTIMODAL_DATASET_NAMES = list(A), list(M)
    return ACTION_DATASET_NAMES + MULTIMODAL_DATASET_NAMES


@dataclass
class Qwen2_5_VLACausalLMOutputWithPast:
    loss: Optional[torch.Tensor] = None
    flow_loss: Optional[torch.Tensor] = None
    cross_entropy_loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    past_key_values: Optional[Any] = None
    hidden_states: Optional[Any] = None
    attentions: Optional[Any] = None
    rope_deltas: Optional[torch.Tensor] = None
    channel_loss_dict: Optional[dict] = None
    channel_loss_count_dict: Optional[dict] = None

    # dict-style access, as HF ModelOutput offers and the trainer uses (`"x" in outputs`)
    def keys(self):
        return [f.name for f in fields(self) if getattr(self, f.name) is not None]

    def __contains__(self, k):
        return k in self.keys()

    def __getitem__(self, k):
        if isinstance(k, str):
            return getattr(self, k)
        return tuple(getattr(self, n) for n in self.keys())[k]

    def get(self, k, default=None):
        v = getattr(self, k, None)
        return default if v is None else v


def replace_rows_where(emb: torch.Tensor, mask: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """``emb[mask] = src`` (rows, in order) without a host sync and differentiable in both."""
    if src.shape[0] == 0:
        return emb
    order = (torch.cumsum(mask.to(torch.int64), 0) - 1).clamp_(0, src.shape[0] - 1)
    return torch.where(mask.unsqueeze(-1), src.index_select(0, order).to(emb.dtype), emb)


class PackInfo:
    """Packing of a padded ``[B, S]`` batch into ``T`` valid tokens."""

    def __init__(self, B: int, S: int, seq_lens: List[int], pack_index: torch.Tensor):
        self.B, self.S = B, S
        self.seq_lens = seq_lens
        self.cu = [0]
        for l in seq_lens:
            self.cu.append(self.cu[-1] + l)
        self.T = self.cu[-1]
        self.pack_index = pack_index

    @staticmethod
    def build(attention_mask: Optional[torch.Tensor], B: int, S: int, device, seq_lens=None, pack_index=None):
        if pack_index is not None and seq_lens is not None:
            lens = [int(x) for x in (seq_lens.tolist() if isinstance(seq_lens, torch.Tensor) else seq_lens)]
            return PackInfo(B, S, lens, pack_index.to(device))
        if attention_mask is None:
            return PackInfo(B, S, [S] * B, torch.arange(B * S, device=device))
        am = attention_mask.to(torch.bool)
        lens = am.sum(1).tolist()  # host sync; avoided when the collator supplies the info
        idx = torch.nonzero(am.reshape(-1), as_tuple=False).squeeze(1).to(device)
        return PackInfo(B, S, [int(l) for l in lens], idx)


class Qwen2_5_VLMoEForAction(GenerationHooksMixin, nn.Module):
    _tied_weights_keys = ["lm_head.weight"]
    config_class = Qwen2_5_VLConfig
    _no_split_modules = ["DecoderLayer", "VisionBlock"]

    # ------------------------------------------------------------------ construction / IO
    @classmethod
    def from_pretrained(cls, pretrained_model_path, config_path=None, processor_path=None, action_tokenizer_path=None,
                        **kwargs):
        """Load ``config.json`` + every ``*.safetensors`` in the directory (HF key layout).

        The processor is taken from ``kwargs['processor']`` when given, else loaded with
        ``transformers.AutoProcessor`` from the same directory (needs the HF processor files)."""
        from ..train.checkpoint import load_safetensors_dir

        config_path = config_path or os.path.join(pretrained_model_path, "config.json")
        config = cls.config_class.from_pretrained(config_path)
        processor = kwargs.pop("processor", None)
        if processor is None:
            from transformers import AutoProcessor

            processor = AutoProcessor.from_pretrained(processor_path or pretrained_model_path, use_fast=True)
        if action_tokenizer_path is not None:
            from transformers import AutoProcessor

            processor.action_processor = AutoProcessor.from_pretrained(action_tokenizer_path, trust_remote_code=True)
        model = cls(config, processor=processor, **kwargs)
        model.resize_token_embeddings(len(processor.tokenizer))
        state = load_safetensors_dir(pretrained_model_path)
        missing, unexpected = model.load_state_dict(state, strict=False)
        model._load_report = {"missing": list(missing), "unexpected": list(unexpected)}
        return model

    def save_pretrained(self, directory: str, max_shard_bytes: int = 4 << 30):
        from ..train.checkpoint import save_safetensors_sharded

        os.makedirs(directory, exist_ok=True)
        self.config.vocab_size = self.model.embed_tokens.weight.shape[0]
        self.config.save_pretrained(directory)
        save_safetensors_sharded(self.state_dict(), directory, max_shard_bytes)

    def __init__(self, config: Qwen2_5_VLConfig, use_fast_tokenizer=False, processor=None, action_tokenizer=None,
                 action_mapper=None, flow_loss_weight=1.0):
        super().__init__()
        self.config = config
        self.visual = VisionTransformer(config.vision_config)
        self.model = Qwen2_5_VLMoEModel(config)
        self.vocab_size = config.vocab_size
        self.lm_head = Linear(config.hidden_size, config.vocab_size, bias=False)
        self.flow_loss_weight = flow_loss_weight
        self.use_fast_tokenizer = use_fast_tokenizer
        self.processor = processor
        self.action_tokenizer = action_tokenizer
        self.action_mapper = action_mapper
        self.action_token_id_set = {"fast_action_token_list": [], "propri_token_id": None, "action_token_id": None}
        if processor is not None:
            self.define_action_token_id()
        self.rope_deltas = None
        self.action_preprocessor = ActionProcessor(config)
        self.init_weights()
        if getattr(config, "use_lora", False):
            self.add_lora(r=config.lora_r, lora_alpha=config.lora_alpha, target_modules=config.lora_target_modules,
                          lora_dropout=config.lora_dropout)

    @torch.no_grad()
    def init_weights(self, seed: Optional[int] = None):
        """normal(0, initializer_range) weights, zero biases, unit RMSNorm weights, zero padding row.

        With ``seed`` the values come from a CPU generator (reproducible across devices); without it
        they are drawn in place on whatever device the parameters live on (fast for large models)."""
        from .layers import FusedQKV, RMSNorm, SwiGLUFFN

        gen = torch.Generator().manual_seed(seed) if seed is not None else None
        std = self.config.initializer_range

        def fill(t: torch.Tensor):
            if gen is None:
                t.normal_(0.0, std)
            else:
                t.copy_(torch.empty(t.shape, dtype=torch.float32).normal_(0.0, std, generator=gen))

        for mod in self.modules():
            if isinstance(mod, SwiGLUFFN):
                if gen is None:
                    fill(mod.gate_up_weight)
                    fill(mod.down_weight)
                    pad = mod.padded - mod.intermediate
                    if pad:  # padding rows / columns must be zero
                        g, u = mod.unpack_gate_up(mod.gate_up_weight.data)
                        mod.gate_up_weight.copy_(mod.pack_gate_up(g, u))
                        mod.down_weight[:, mod.intermediate:].zero_()
                    if mod.gate_up_bias is not None:
                        mod.gate_up_bias.zero_()
                        mod.down_bias.zero_()
                else:
                    mod.reset_parameters(std, gen)
            elif isinstance(mod, (Linear, FusedQKV)):
                fill(mod.weight)
                if mod.bias is not None:
                    mod.bias.zero_()
            elif isinstance(mod, nn.Embedding):
                fill(mod.weight)
                if mod.padding_idx is not None:
                    mod.weight[mod.padding_idx].zero_()
            elif isinstance(mod, RMSNorm):
                mod.weight.fill_(1.0)
        fill(self.visual.patch_embed.proj.weight)

    def define_action_token_id(self):
        tok = self.processor.tokenizer
        fast = [tok.convert_tokens_to_ids(f"<|action_token_{i}|>")
                for i in range(tok.init_kwargs.get("action_token_vocab_size", 0))]
        self.action_token_id_set = {
            "fast_action_token_list": fast,
            "propri_token_id": tok.convert_tokens_to_ids("<|propri|>"),
            "action_token_id": tok.convert_tokens_to_ids("<|action|>"),
        }

    def add_lora(self, r=8, lora_alpha=32, target_modules=("q_proj", "v_proj"), lora_dropout=0.1):
        from .lora import apply_lora

        n = apply_lora(self.model, r=r, alpha=lora_alpha, target_modules=list(target_modules), dropout=lora_dropout)
        print(f"LoRA: wrapped {n} projections (r={r}, alpha={lora_alpha})")

    def resize_token_embeddings(self, new_num_tokens: int):
        old = self.model.embed_tokens.weight
        if new_num_tokens == old.shape[0]:
            return self.model.embed_tokens
        std = self.config.initializer_range
        for holder, name in ((self.model.embed_tokens, "weight"), (self.lm_head, "weight")):
            w = getattr(holder, name)
            nw = torch.empty((new_num_tokens, w.shape[1]), dtype=w.dtype, device=w.device).normal_(0.0, std)
            n = min(new_num_tokens, w.shape[0])
            nw[:n] = w.data[:n]
            setattr(holder, name, nn.Parameter(nw))
        self.model.embed_tokens.num_embeddings = new_num_tokens
        self.lm_head.out_features = new_num_tokens
        self.config.vocab_size = new_num_tokens
        self.vocab_size = new_num_tokens
        self.model.vocab_size = new_num_tokens
        return self.model.embed_tokens

    # ------------------------------------------------------------------ small accessors
    def get_input_embeddings(self):
        return self.model.embed_tokens

    def set_input_embeddings(self, value):
        self.model.embed_tokens = value

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, new_embeddings):
        self.lm_head = new_embeddings

    def set_decoder(self, decoder):
        self.model = decoder

    def get_decoder(self):
        return self.model

    def enable_input_require_grads(self):
        def hook(module, inputs, output):
            output.requires_grad_(True)

        self._require_grads_hook = self.model.embed_tokens.register_forward_hook(hook)

    @property
    def device(self):
        return self.lm_head.weight.device

    @property
    def dtype(self):
        return self.lm_head.weight.dtype

    def get_rope_index(self, input_ids=None, image_grid_thw=None, video_grid_thw=None, second_per_grid_ts=None,
                       attention_mask=None):
        vc = self.config.vision_config
        return IX.get_rope_index(input_ids, image_grid_thw, video_grid_thw, second_per_grid_ts, attention_mask,
                                 vc.spatial_merge_size, self.config.image_token_id, self.config.video_token_id,
                                 self.config.vision_start_token_id, vc.tokens_per_second)

    # ------------------------------------------------------------------ embedding assembly
    def _embed_packed(self, ids, pack: PackInfo, pixel_values, image_grid_thw, pixel_values_videos, video_grid_thw,
                      proprioception, agent_pos_mask, dataset_names, image_grid_host=None, video_grid_host=None):
        emb = self.model.embed_tokens(ids)
        if pixel_values is not None:
            img = self.visual(pixel_values.to(self.visual.dtype), image_grid_thw, grid_host=image_grid_host)
            emb = replace_rows_where(emb, ids == self.config.image_token_id, img)
        if pixel_values_videos is not None:
            vid = self.visual(pixel_values_videos.to(self.visual.dtype), video_grid_thw, grid_host=video_grid_host)
            emb = replace_rows_where(emb, ids == self.config.video_token_id, vid)
        if proprioception is not None:
            pe = self.action_preprocessor.proprioception_proj(
                proprioception.to(emb.device, emb.dtype), dataset_names,
                agent_pos_mask.to(emb.device, emb.dtype) if agent_pos_mask is not None else None,
                use_history=proprioception.shape[1] > 1)
            emb = replace_rows_where(emb, ids == self.action_token_id_set["propri_token_id"], pe.reshape(-1, emb.shape[-1]))
        return emb

    def _positions(self, input_ids, position_ids, attention_mask, image_grid_thw, video_grid_thw, second_per_grid_ts):
        if position_ids is not None:
            if position_ids.dim() == 2:
                position_ids = position_ids.unsqueeze(0).expand(3, -1, -1)
            return position_ids, self.rope_deltas
        pos, deltas = self.get_rope_index(input_ids, image_grid_thw, video_grid_thw, second_per_grid_ts, attention_mask)
        self.rope_deltas = deltas
        return pos.to(input_ids.device), deltas

    # ------------------------------------------------------------------ training / validation forward
    def train_step_forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None,
                           inputs_embeds=None, moe_token_types=None, labels=None, use_cache=None,
                           output_attentions=None, output_hidden_states=None, return_dict=None, pixel_values=None,
                           pixel_values_videos=None, image_grid_thw=None, video_grid_thw=None, action_chunk=None,
                           proprioception=None, rope_deltas=None, cache_position=None, second_per_grid_ts=None,
                           dataset_names=None, dof_mask=None, agent_pos_mask=None, return_logits=None, pack_index=None,
                           seq_lens=None, label_index=None, image_grid_host=None, video_grid_host=None,
                           flow_noise=None, flow_time=None, generator=None, **kwargs):
        B, S = input_ids.shape
        dev = self.model.embed_tokens.weight.device
        input_ids = input_ids.to(dev)
        if moe_token_types is None:
            moe_token_types = torch.zeros_like(input_ids)
        moe_token_types = moe_token_types.to(dev)
        if attention_mask is not None:
            attention_mask = attention_mask.to(dev)
        position_ids, deltas = self._positions(input_ids, position_ids.to(dev) if position_ids is not None else None,
                                               attention_mask, image_grid_thw, video_grid_thw, second_per_grid_ts)
        pack = PackInfo.build(attention_mask, B, S, dev, seq_lens, pack_index)
        ids = input_ids.reshape(-1).index_select(0, pack.pack_index)
        types = moe_token_types.reshape(-1).index_select(0, pack.pack_index).to(torch.int32)
        pos3 = position_ids.reshape(3, -1).index_select(1, pack.pack_index)

        if inputs_embeds is None:
            emb = self._embed_packed(ids, pack, pixel_values, image_grid_thw, pixel_values_videos, video_grid_thw,
                                     proprioception, agent_pos_mask, dataset_names, image_grid_host, video_grid_host)
        else:
            emb = inputs_embeds.reshape(B * S, -1).index_select(0, pack.pack_index)

        flow = None
        action_id = self.action_token_id_set["action_token_id"]
        if action_chunk is not None:
            action_chunk = action_chunk.to(dev, emb.dtype)
            dof_mask = dof_mask.to(dev, emb.dtype)
            a_emb, flow = self.action_preprocessor(action_chunk, dataset_names, dof_mask, noise=flow_noise,
                                                   time=flow_time, generator=generator)
            emb = replace_rows_where(emb, ids == action_id, a_emb.reshape(-1, emb.shape[-1]))

        bidir = (types == 1) if self.config.action_attn == "bidirectional" else None
        meta = F_.AttnMeta(pack.cu, dev, causal=True, bidir_q=bidir)
        cos, sin = self.model.rotary(pos3)
        plan = F_.make_route_plan(types, self.config.num_experts) if self.config.mlp_moe else None
        ctx = StepContext(meta, cos, sin, plan)
        hidden = self.model(emb, ctx)  # [T, H]

        loss = None
        ce_loss = flow_loss = None
        channel_loss_dict = channel_loss_count_dict = None
        logits = None
        want_logits = return_logits if return_logits is not None else False

        if labels is not None:
            labels = labels.to(dev)
            shift = torch.cat([labels[:, 1:], labels.new_full((B, 1), -100)], dim=1).reshape(-1)
            shift = shift.index_select(0, pack.pack_index)  # label of the *next* token, per packed row
            # a row's successor must belong to the same sequence: the last token of a sequence has none
            last = torch.tensor([c - 1 for c in pack.cu[1:]], device=dev, dtype=torch.long)
            if attention_mask is not None and len(last):
                shift = shift.clone()
                shift[last] = -100
            if label_index is not None:
                rows = label_index.to(dev)
            else:
                rows = torch.nonzero(shift != -100, as_tuple=False).squeeze(1)  # host sync (collator can supply it)
            sel_labels = shift.index_select(0, rows)
            if rows.numel() > 0:
                tok_loss, pred = F_.lm_head_ce(hidden.index_select(0, rows), self.lm_head.weight, sel_labels)
                valid = (sel_labels != -100).float()
                ce_loss = (tok_loss * valid).sum() / valid.sum().clamp_min(1.0)
            else:
                tok_loss = hidden.new_zeros((0,), dtype=torch.float32)
                pred = sel_labels
                valid = tok_loss
                ce_loss = hidden.new_zeros((), dtype=torch.float32)
            names = list(dataset_names) if dataset_names is not None else ["x2_normal"] * B
            channel_loss_dict = {n: torch.zeros((), device=dev) for n in _dataset_names()}
            channel_loss_count_dict = {n: torch.zeros((), device=dev, dtype=torch.long) for n in _dataset_names()}
            sample_of_tok = torch.repeat_interleave(torch.arange(B, device=dev),
                                                    torch.tensor(pack.seq_lens, device=dev), output_size=pack.T)
            samp = sample_of_tok.index_select(0, rows)
            per_sample = torch.zeros(B, device=dev).index_add_(0, samp, (tok_loss * valid).detach())
            per_count = torch.zeros(B, device=dev).index_add_(0, samp, valid)
            for name in set(names):
                m = torch.tensor([n == name for n in names], device=dev)
                channel_loss_dict[name] = (per_sample * m).sum()
                channel_loss_count_dict[name] = channel_loss_count_dict.get(
                    name, torch.zeros((), device=dev, dtype=torch.long)) + (per_count * m).sum().long()
            loss = ce_loss
            if self.use_fast_tokenizer and self.action_token_id_set["fast_action_token_list"]:
                amask = sel_labels > self.action_token_id_set["fast_action_token_list"][0]
                correct = ((pred == sel_labels) & amask).sum().float()
                channel_loss_dict["action_accuracy"] = correct / amask.sum().float()

        if action_chunk is not None and flow is not None:
            n_act = flow.shape[0] * flow.shape[1]
            amask = ids == action_id
            arow = torch.nonzero_static(amask, size=n_act, fill_value=0).squeeze(1) if hasattr(torch, "nonzero_static") \
                else torch.nonzero(amask).squeeze(1)
            a_hidden = hidden.index_select(0, arow)
            fl = self.action_preprocessor.flow_loss(a_hidden, flow.reshape(-1, flow.shape[-1]), dof_mask)
            flow_loss = fl.mean()
            loss = self.flow_loss_weight * flow_loss if loss is None else loss + self.flow_loss_weight * flow_loss

        if want_logits:
            full = F_.linear(hidden, self.lm_head.weight)
            logits = full.new_zeros((B * S, full.shape[-1]))
            logits.index_copy_(0, pack.pack_index, full)
            logits = logits.view(B, S, -1)

        return Qwen2_5_VLACausalLMOutputWithPast(
            loss=loss, cross_entropy_loss=ce_loss.detach().clone() if ce_loss is not None else None, flow_loss=flow_loss,
            logits=logits, past_key_values=None, hidden_states=None, attentions=None, rope_deltas=deltas,
            channel_loss_dict=channel_loss_dict, channel_loss_count_dict=channel_loss_count_dict)

    # ------------------------------------------------------------------ inference
    def predict_action(self, predict_mode: str, **kwargs):
        assert predict_mode in ["text", "fast", "diffusion"]
        return self.predict(predict_mode=predict_mode, **kwargs)

    @torch.no_grad()
    def predict(self, predict_mode: str, pred_horizon=None, action_dim=None, input_ids=None, attention_mask=None,
                position_ids=None, past_key_values=None, inputs_embeds=None, moe_token_types=None, labels=None,
                use_cache=None, pixel_values=None, pixel_values_videos=None, image_grid_thw=None, video_grid_thw=None,
                action_chunk=None, proprioception=None, rope_deltas=None, cache_position=None,
                second_per_grid_ts=None, num_inference_timesteps=10, dataset_names=None, dof_mask=None,
                agent_pos_mask=None, re_generate=False, image_grid_host=None, video_grid_host=None, noise=None,
                reference_grid=False, use_cuda_graph=False, **kwargs):
        from . import inference as INF

        if predict_mode == "diffusion":
            return INF.predict_flow(self, pred_horizon=pred_horizon, action_dim=action_dim, input_ids=input_ids,
                                    attention_mask=attention_mask, position_ids=position_ids,
                                    moe_token_types=moe_token_types, pixel_values=pixel_values,
                                    pixel_values_videos=pixel_values_videos, image_grid_thw=image_grid_thw,
                                    video_grid_thw=video_grid_thw, action_chunk=action_chunk,
                                    proprioception=proprioception, second_per_grid_ts=second_per_grid_ts,
                                    num_inference_timesteps=num_inference_timesteps, dataset_names=dataset_names,
                                    dof_mask=dof_mask, agent_pos_mask=agent_pos_mask, image_grid_host=image_grid_host,
                                    video_grid_host=video_grid_host, noise=noise, reference_grid=reference_grid,
                                    use_cuda_graph=use_cuda_graph)
        if predict_mode in ("text", "fast"):
            assert input_ids.shape[0] == 1, "predict only support batch size 1 for ar generation"
            return INF.predict_text(self, predict_mode, pred_horizon=pred_horizon, action_dim=action_dim,
                                    input_ids=input_ids, attention_mask=attention_mask, pixel_values=pixel_values,
                                    image_grid_thw=image_grid_thw, action_chunk=action_chunk,
                                    proprioception=proprioception, dataset_names=dataset_names, dof_mask=dof_mask,
                                    agent_pos_mask=agent_pos_mask, re_generate=re_generate, labels=labels,
                                    image_grid_host=image_grid_host)
        raise NotImplementedError(predict_mode)

    @torch.no_grad()
    def generate(self, input_ids=None, max_new_tokens: int = 100, do_sample: bool = False, temperature: float = 1.0,
                 eos_token_id=None, pad_token_id=None, use_cache: bool = True, **kwargs):
        from . import inference as INF

        return INF.generate(self, input_ids, max_new_tokens=max_new_tokens, do_sample=do_sample,
                            temperature=temperature, eos_token_id=eos_token_id, pad_token_id=pad_token_id, **kwargs)

    def forward(self, mode: Optional[str] = None, predict_mode: Optional[str] = "text", **kwargs):
        if not mode:
            with torch.no_grad():
                kwargs.setdefault("return_logits", True)
                return self.train_step_forward(**kwargs)
        if mode == "predict":
            return self.predict(predict_mode=predict_mode, **kwargs)
        if mode == "train":
            return self.train_step_forward(use_cache=False, **kwargs)
        if mode == "validate":
            with torch.no_grad():
                kwargs.setdefault("return_logits", True)
                return self.train_step_forward(use_cache=False, **kwargs)
        raise NotImplementedError("invalid key")

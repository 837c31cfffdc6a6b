"""Tiny VLA model on CPU: losses, state-dict layout, checkpoint round trip, inference parity."""
import copy
import os

import pytest
import torch

from wallx_b200.config import Qwen2_5_VLConfig, tiny_config
from wallx_b200.data.collator import add_pack_info
from wallx_b200.data.synthetic import make_batch, make_processor
from wallx_b200.models import Qwen2_5_VLMoEForAction
from wallx_b200.ops import functional as F_


@pytest.fixture(scope="module")
def setup():
    cfg = tiny_config()
    proc = make_processor(cfg, 16)
    torch.manual_seed(0)
    model = Qwen2_5_VLMoEForAction(cfg, processor=proc)
    model.init_weights(seed=3)
    return cfg, proc, model


def _flow_batch(cfg, proc, B=2, seed=1):
    g = torch.Generator().manual_seed(seed)
    return add_pack_info(make_batch(cfg, proc, B, views=1, image_hw=(112, 112), prompt_len=16, horizon=16, mode="flow",
                                    generator=g), cfg)


def test_flow_forward_backward_is_reproducible(setup):
    cfg, proc, model = setup
    batch = _flow_batch(cfg, proc)
    outs = []
    for _ in range(2):
        model.zero_grad()
        out = model(mode="train", generator=torch.Generator().manual_seed(7), **batch)
        out.loss.backward()
        outs.append((out.loss.item(), model.model.layers[0].moe.experts[1].gate_up_weight.grad.norm().item()))
    assert outs[0] == outs[1]
    assert out.cross_entropy_loss is None and out.flow_loss is not None and torch.isfinite(out.loss)
    assert model.lm_head.weight.grad is None  # flow mode never touches the LM head
    for n in ("visual.blocks.0.attn.qkv.weight", "model.layers.1.self_attn.qkv_proj.weight",
              "action_preprocessor.w1.weight", "action_preprocessor.propri_proj.weight"):
        p = dict(model.named_parameters())[n]
        assert p.grad is not None and p.grad.abs().sum() > 0, n


def test_fast_mode_cross_entropy_and_metrics(setup):
    cfg, proc, _ = setup
    torch.manual_seed(1)
    model = Qwen2_5_VLMoEForAction(cfg, processor=proc, use_fast_tokenizer=True)
    batch = add_pack_info(make_batch(cfg, proc, 3, views=1, image_hw=(112, 112), prompt_len=16, mode="fast",
                                     fast_tokens=12, generator=torch.Generator().manual_seed(2)), cfg)
    out = model(mode="train", return_logits=True, **batch)
    assert out.flow_loss is None and out.cross_entropy_loss is not None
    # oracle: full logits, shifted CE over labelled positions
    logits = out.logits[:, :-1].reshape(-1, out.logits.shape[-1]).float()
    labels = batch["labels"][:, 1:].reshape(-1)
    ce = torch.nn.functional.cross_entropy(logits, labels, ignore_index=-100)
    assert abs(ce.item() - out.cross_entropy_loss.item()) < 1e-4
    assert "action_accuracy" in out.channel_loss_dict
    cnt = out.channel_loss_count_dict["x2_normal"].item()
    assert cnt == (labels != -100).sum().item()
    assert abs(out.channel_loss_dict["x2_normal"].item() / cnt - ce.item()) < 1e-4
    out.loss.backward()
    assert model.lm_head.weight.grad.abs().sum() > 0
    assert "loss" in out and out["loss"] is out.loss


def test_padding_invariance(setup):
    """Left padding must not change the result (padding rows never enter a kernel)."""
    cfg, proc, model = setup
    g = torch.Generator().manual_seed(5)
    b1 = make_batch(cfg, proc, 2, views=1, image_hw=(112, 112), prompt_len=16, horizon=16, generator=g)
    g = torch.Generator().manual_seed(5)
    b2 = make_batch(cfg, proc, 2, views=1, image_hw=(112, 112), prompt_len=16, horizon=16, generator=g, pad_to=80)
    assert b2["input_ids"].shape[1] == 80 and b1["input_ids"].shape[1] < 80
    noise = torch.randn(b1["action_chunk"].shape)
    t = torch.tensor([0.3, 0.7])
    l1 = model(mode="validate", flow_noise=noise, flow_time=t, **add_pack_info(b1, cfg)).loss
    l2 = model(mode="validate", flow_noise=noise, flow_time=t, **add_pack_info(b2, cfg)).loss
    l3 = model(mode="validate", flow_noise=noise, flow_time=t, **{k: v for k, v in b2.items() if k not in
                                                                   ("pack_index", "seq_lens", "position_ids")}).loss
    assert abs(l1.item() - l2.item()) < 1e-5 and abs(l1.item() - l3.item()) < 1e-5


def test_state_dict_uses_reference_key_layout(setup):
    _, _, model = setup
    keys = set(model.state_dict().keys())
    for k in ["visual.patch_embed.proj.weight", "visual.blocks.0.norm1.weight", "visual.blocks.0.attn.qkv.weight",
              "visual.blocks.0.attn.qkv.bias", "visual.blocks.0.attn.proj.bias", "visual.blocks.1.mlp.gate_proj.bias",
              "visual.blocks.1.mlp.down_proj.weight", "visual.merger.ln_q.weight", "visual.merger.mlp.0.weight",
              "visual.merger.mlp.2.bias", "model.embed_tokens.weight", "model.layers.0.input_layernorm.weight",
              "model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.k_proj.bias",
              "model.layers.0.self_attn.v_proj.weight", "model.layers.0.self_attn.o_proj.weight",
              "model.layers.1.moe.experts.0.gate_proj.weight", "model.layers.1.moe.experts.1.down_proj.weight",
              "model.norm.weight", "lm_head.weight", "action_preprocessor.w1.weight", "action_preprocessor.w2.weight",
              "action_preprocessor.w3.weight", "action_preprocessor.propri_proj.weight",
              "action_preprocessor.action_proj_back.weight", "action_preprocessor.normalizer_action.min.x2_normal",
              "action_preprocessor.normalizer_propri.delta.DobbE"]:
        assert k in keys, k
    assert not any("qkv_proj" in k or "gate_up" in k for k in keys)
    sd = model.state_dict()
    assert sd["visual.patch_embed.proj.weight"].shape == (128, 3, 2, 14, 14)
    assert sd["model.layers.0.moe.experts.1.gate_proj.weight"].shape == (256, 256)
    assert sd["visual.blocks.0.mlp.up_proj.weight"].shape == (256, 128)


def test_save_and_from_pretrained_round_trip(setup, tmp_path):
    cfg, proc, model = setup
    d = str(tmp_path / "ckpt")
    model.save_pretrained(d, max_shard_bytes=1 << 20)  # forces several shards + index
    assert os.path.exists(os.path.join(d, "model.safetensors.index.json"))
    m2 = Qwen2_5_VLMoEForAction.from_pretrained(d, processor=proc)
    assert not m2._load_report["missing"] and not m2._load_report["unexpected"]
    batch = _flow_batch(cfg, proc)
    noise = torch.randn(batch["action_chunk"].shape)
    t = torch.tensor([0.2, 0.9])
    a = model(mode="validate", flow_noise=noise, flow_time=t, **batch)
    b = m2(mode="validate", flow_noise=noise, flow_time=t, **batch)
    assert torch.equal(a.logits, b.logits) and a.loss.item() == b.loss.item()
    c2 = Qwen2_5_VLConfig.from_pretrained(d)
    assert c2.experts == cfg.experts and c2.mrope_section == cfg.mrope_section


def test_vit_intermediate_padding_is_transparent():
    cfg = tiny_config(vision_config=dict(depth=1, hidden_size=128, intermediate_size=200, num_heads=4, patch_size=14,
                                         spatial_merge_size=2, temporal_patch_size=2, window_size=112,
                                         out_hidden_size=256, fullatt_block_indexes=[0]))
    proc = make_processor(cfg, 16)
    m = Qwen2_5_VLMoEForAction(cfg, processor=proc)
    ffn = m.visual.blocks[0].mlp
    assert ffn.padded == 256 and ffn.gate_up_weight.shape == (512, 128)
    sd = m.state_dict()
    assert sd["visual.blocks.0.mlp.gate_proj.weight"].shape == (200, 128)
    assert sd["visual.blocks.0.mlp.down_proj.weight"].shape == (128, 200)
    m2 = Qwen2_5_VLMoEForAction(cfg, processor=proc)
    m2.load_state_dict(sd)
    x = torch.randn(5, 128)
    assert torch.allclose(m.visual.blocks[0].mlp(x), m2.visual.blocks[0].mlp(x))
    g, u = ffn.unpack_gate_up(ffn.gate_up_weight.data)
    ref_out = torch.nn.functional.linear(torch.nn.functional.silu(x @ g.t()) * (x @ u.t()), ffn.down_weight[:, :200], ffn.down_bias)
    assert torch.allclose(ffn(x), ref_out, atol=1e-5)


def test_qwen_rename_and_resize_embeddings(setup):
    from wallx_b200.train.checkpoint import rename_qwen_to_moe, strip_prefixes

    sd = {"model.layers.3.mlp.gate_proj.weight": torch.zeros(1), "visual.blocks.0.mlp.up_proj.weight": torch.zeros(1),
          "model.norm.weight": torch.zeros(1)}
    out = rename_qwen_to_moe(sd)
    assert "model.layers.3.moe.experts.0.gate_proj.weight" in out and "visual.blocks.0.mlp.up_proj.weight" in out
    assert list(strip_prefixes({"module._orig_mod.a.b": 1}).keys()) == ["a.b"]
    cfg, proc, _ = setup
    cfg2 = copy.deepcopy(cfg)
    v0 = cfg2.vocab_size
    m = Qwen2_5_VLMoEForAction(cfg2, processor=proc)
    old = m.model.embed_tokens.weight.data.clone()
    m.resize_token_embeddings(v0 + 10)
    assert m.model.embed_tokens.weight.shape[0] == v0 + 10 == m.lm_head.weight.shape[0] == m.config.vocab_size
    assert torch.equal(m.model.embed_tokens.weight.data[:v0], old)


def test_flow_sampler_with_prefix_cache_equals_full_recompute(setup):
    """Euler sampling with the reused prefix KV must equal re-running the whole sequence each step."""
    from wallx_b200.models.inference import FlowSampler
    from wallx_b200.models.llm import StepContext
    from wallx_b200.models.vla import PackInfo, replace_rows_where

    cfg, proc, model = setup
    model.eval()
    batch = _flow_batch(cfg, proc, B=2, seed=9)
    B = 2
    noise = torch.randn(B, 16, 14, generator=torch.Generator().manual_seed(4))
    keys = ("input_ids", "attention_mask", "position_ids", "moe_token_types", "pixel_values", "image_grid_thw",
            "proprioception", "agent_pos_mask", "dataset_names", "dof_mask", "image_grid_host", "pack_index", "seq_lens")
    sampler = FlowSampler(model, **{k: batch[k] for k in keys})
    n = 4
    # the host knows that the suffix rows are all action tokens and the prefix rows are not: both passes run one expert as
    # a plain FFN, and the comparison below is against the grouped two-expert path
    assert sampler.ctx.plan.single_expert == 1 and sampler.ctx_pre.plan.single_expert == 0
    x_fast = sampler.sample(noise, num_steps=n)

    # oracle: full sequence every evaluation (the reference's procedure)
    with torch.no_grad():
        ids2d = batch["input_ids"]
        pack = PackInfo.build(batch["attention_mask"], B, ids2d.shape[1], "cpu", batch["seq_lens"], batch["pack_index"])
        ids = ids2d.reshape(-1)[pack.pack_index]
        types = batch["moe_token_types"].reshape(-1)[pack.pack_index].to(torch.int32)
        pos3 = batch["position_ids"].reshape(3, -1)[:, pack.pack_index]
        emb = model._embed_packed(ids, pack, batch["pixel_values"], batch["image_grid_thw"], None, None,
                                  batch["proprioception"], batch["agent_pos_mask"], batch["dataset_names"],
                                  batch["image_grid_host"])
        act = ids == model.action_token_id_set["action_token_id"]
        meta = F_.AttnMeta(pack.cu, "cpu", True, bidir_q=(types == 1))
        cos, sin = model.model.rotary(pos3)
        plan = F_.make_route_plan(types, cfg.num_experts)
        x = noise.clone()
        ts = torch.linspace(0, 1, n + 1)
        for i in range(n):
            a_emb = model.action_preprocessor.step(ts[i].reshape(1).expand(B), x, batch["dof_mask"]).reshape(B * 16, -1)
            h = model.model(replace_rows_where(emb, act, a_emb), StepContext(meta, cos, sin, plan))
            v = model.action_preprocessor.action_proj_back(h[act]).reshape(B, 16, 14)
            x = x + (ts[i + 1] - ts[i]) * v
    assert torch.allclose(x_fast, x, atol=2e-4), (x_fast - x).abs().max()
    out = model(mode="predict", predict_mode="diffusion", num_inference_timesteps=n, noise=noise,
                **{k: batch[k] for k in keys}, action_chunk=batch["action_chunk"])
    assert out["predict_action"].shape == (B, 16, 14) and out["gt_action"].shape == (B, 16, 14)
    un = model.action_preprocessor.normalizer_action.unnormalize_data(x_fast.float(), batch["dataset_names"])
    assert torch.allclose(out["predict_action"], un, atol=1e-5)
    ref_grid = sampler.sample(noise, num_steps=n, reference_grid=True)  # linspace(0,1,n): n-1 evaluations
    assert not torch.allclose(ref_grid, x_fast)


def test_greedy_generate_matches_full_forward(setup):
    cfg, proc, model = setup
    model.eval()
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(6, 900, (2, 9), generator=g)
    am = torch.ones_like(ids)
    am[0, :3] = 0  # left padding on the first prompt
    out = model.generate(input_ids=ids, attention_mask=am, max_new_tokens=4, eos_token_id=None)
    assert out.shape == (2, 13)
    cur, cam = ids.clone(), am.clone()
    for _ in range(4):  # oracle: recompute everything, take the argmax at the last position
        lg = model(mode="validate", input_ids=cur, attention_mask=cam, moe_token_types=torch.zeros_like(cur)).logits
        nxt = lg[:, -1].argmax(-1, keepdim=True)
        cur = torch.cat([cur, nxt], 1)
        cam = torch.cat([cam, torch.ones_like(nxt)], 1)
    assert torch.equal(out, cur)


def test_lora_freezes_base_and_trains_adapters(setup):
    cfg, proc, _ = setup
    m = Qwen2_5_VLMoEForAction(cfg, processor=proc)
    m.add_lora(r=4, lora_alpha=8, target_modules=["q_proj", "v_proj", "o_proj"], lora_dropout=0.0)
    names = [n for n, p in m.model.named_parameters() if p.requires_grad]
    assert names and all("lora_" in n for n in names)
    batch = _flow_batch(cfg, proc)
    out = m(mode="train", **batch)
    out.loss.backward()
    got = [n for n, p in m.model.named_parameters() if p.requires_grad and p.grad is not None]
    assert len(got) == len(names)


def test_flow_engine_matches_predict_on_cpu():
    """FlowEngine without a graph (CPU): identical to ``predict`` for the same noise; a changed
    placeholder layout is refused."""
    import copy

    from wallx_b200.config import tiny_config
    from wallx_b200.data.collator import add_pack_info
    from wallx_b200.data.synthetic import make_batch, make_processor
    from wallx_b200.models import Qwen2_5_VLMoEForAction
    from wallx_b200.models.inference import FlowEngine

    cfg = tiny_config()
    proc = make_processor(cfg, 16)
    torch.manual_seed(0)
    model = Qwen2_5_VLMoEForAction(cfg, processor=proc).float().eval()
    batch = make_batch(cfg, proc, 2, views=1, image_hw=(112, 112), prompt_len=16, horizon=8, mode="flow",
                       generator=torch.Generator().manual_seed(1))
    inp = {k: v for k, v in batch.items() if k not in ("action_chunk", "labels")}
    A = model.action_preprocessor.action_dim
    noise = torch.randn(2, 8, A)
    eng = FlowEngine(model, inp, num_inference_timesteps=3)
    new = dict(inp)
    new["proprioception"] = torch.randn_like(inp["proprioception"])
    ref = model(mode="predict", predict_mode="diffusion", noise=noise, num_inference_timesteps=3, **new)
    got = eng(new, noise=noise)
    assert torch.equal(ref["predict_action"], got["predict_action"])
    bad = dict(inp)
    ids = inp["input_ids"].clone()
    ids[0, 3] = cfg.image_token_id
    bad["input_ids"] = ids
    with pytest.raises(ValueError):
        eng(bad)


def test_dense_mask_rule_equals_the_interval_rule_of_the_kernels(setup):
    """The reference-named dense mask builder and the varlen rule the attention kernels implement agree."""
    from wallx_b200.ops import ref

    cfg, proc, model = setup
    B, S, C = 2, 9, 4
    x = torch.zeros(B, S, C)
    types = torch.zeros(B, S, dtype=torch.long)
    types[0, 5:8] = 1
    types[1, 6:9] = 1
    am = torch.ones(B, S, dtype=torch.long)
    am[1, :2] = 0  # left padding
    mask = model.model._update_causal_mask(am, x, torch.arange(S), None, False, moe_token_types=types)
    assert mask.shape == (B, 1, S, S)
    for b in range(B):
        keep = am[b] == 1
        n = int(keep.sum())
        want = ref.attention_mask_varlen([0, n], True, (types[b][keep] == 1), "cpu")
        got = (mask[b, 0] == 0)[keep][:, keep]
        assert torch.equal(got, want)
        assert not (mask[b, 0] == 0)[:, ~keep].any()  # nothing attends to padding
    # decoding step: one query at position 9 sees everything before it
    step = model.model._prepare_4d_causal_attention_mask_with_cache_position(None, 1, 10, torch.float32, "cpu", torch.tensor([9]), B)
    assert step.shape == (B, 1, 1, 10) and (step == 0).all()


def test_generation_hooks(setup):
    cfg, proc, model = setup

    class Past:
        def __init__(self, n):
            self.n = n

        def get_seq_length(self):
            return self.n

    ids = torch.tensor([[5, cfg.vision_start_token_id, cfg.image_token_id, cfg.image_token_id, 7, 8],
                        [cfg.vision_start_token_id, cfg.image_token_id, cfg.vision_start_token_id, cfg.image_token_id, 9, 9]])
    pix = torch.randn(12, 6)
    first = model.prepare_inputs_for_generation(ids, past_key_values=Past(0), pixel_values=pix, cache_position=torch.arange(6))
    assert first["pixel_values"] is pix and torch.equal(first["input_ids"], ids)
    assert first["moe_token_types"].shape == ids.shape and not first["moe_token_types"].any()
    grown = torch.cat([ids, torch.tensor([[3], [4]])], dim=1)
    later = model.prepare_inputs_for_generation(grown, past_key_values=Past(6), pixel_values=pix, cache_position=torch.tensor([6]),
                                                moe_token_types=torch.zeros_like(ids))
    assert later["pixel_values"] is None and later["input_ids"].tolist() == [[3], [4]]
    assert later["moe_token_types"].shape == (2, 1)
    img_n, vid_n = model._get_image_nums_and_video_nums(ids)
    assert img_n.tolist() == [1, 2] and vid_n.tolist() == [0, 0]
    grid = torch.tensor([[1, 2, 2], [1, 2, 2], [1, 2, 2]])  # 4 patches each: sample 0 owns 4 rows, sample 1 owns 8
    ids2, kw = model._expand_inputs_for_generation(2, input_ids=ids, pixel_values=pix, image_grid_thw=grid,
                                                   attention_mask=torch.ones_like(ids), dataset_names=["a", "b"])
    assert ids2.shape == (4, 6) and torch.equal(ids2[0], ids2[1]) and torch.equal(ids2[2], ids[1])
    assert kw["pixel_values"].shape == (24, 6) and torch.equal(kw["pixel_values"][:4], kw["pixel_values"][4:8])
    assert torch.equal(kw["pixel_values"][8:16], pix[4:12]) and kw["image_grid_thw"].shape == (6, 3)
    assert kw["attention_mask"].shape == (4, 6) and kw["dataset_names"] == ["a", "a", "b", "b"]


def test_decoder_stack_from_pretrained(setup, tmp_path):
    from wallx_b200.models.llm import Qwen2_5_VLMoEModel

    cfg, proc, model = setup
    model.save_pretrained(str(tmp_path))
    stack = Qwen2_5_VLMoEModel.from_pretrained(str(tmp_path))
    assert not stack._load_report["missing"]
    for (n1, p1), (n2, p2) in zip(model.model.state_dict().items(), stack.state_dict().items()):
        assert n1 == n2 and torch.equal(p1, p2), n1

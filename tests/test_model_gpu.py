"""Tiny VLA model: GPU bf16 kernels path vs CPU fp32 oracle path (same weights, same noise)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(mode):
    from wallx_b200.config import tiny_config
    from wallx_b200.data.collator import add_pack_info
    from wallx_b200.data.synthetic import make_batch, make_processor
    from wallx_b200.models import Qwen2_5_VLMoEForAction

    cfg = tiny_config()
    proc = make_processor(cfg, 16)
    torch.manual_seed(0)
    model = Qwen2_5_VLMoEForAction(cfg, processor=proc, use_fast_tokenizer=(mode == "fast"))
    g = torch.Generator().manual_seed(1)
    batch = make_batch(cfg, proc, 3, views=2, image_hw=(112, 112), prompt_len=16, horizon=16, mode=mode,
                       fast_tokens=12, generator=g)
    batch = add_pack_info(batch, cfg)
    return cfg, model, batch


@pytest.mark.parametrize("mode", ["flow", "fast"])
def test_tiny_model_gpu_matches_cpu(mode):
    from wallx_b200.data.collator import to_device
    from wallx_b200.ops import gemm as G

    cfg, model, batch = _build(mode)
    model_g = copy.deepcopy(model).to(torch.bfloat16).cuda()
    model_c = copy.deepcopy(model_g).float().cpu()  # identical (bf16-rounded) weights
    extra = {}
    if mode == "flow":
        gen = torch.Generator().manual_seed(2)
        extra["flow_noise"] = torch.randn(batch["action_chunk"].shape, generator=gen)
        extra["flow_time"] = torch.rand(batch["action_chunk"].shape[0], generator=gen) * 0.9
    out_c = model_c(mode="train", **batch, **extra)
    out_c.loss.backward()
    bg = to_device(batch, "cuda", torch.bfloat16)
    eg = {k: v.cuda() for k, v in extra.items()}
    out_g = model_g(mode="train", **bg, **eg)
    out_g.loss.backward()
    torch.cuda.synchronize()
    G.check_status()
    lc, lg = out_c.loss.item(), out_g.loss.item()
    assert abs(lc - lg) / max(abs(lc), 1e-3) < 0.03, (lc, lg)
    # gradients: compare the direction of a few large tensors
    pc = dict(model_c.named_parameters())
    checked = 0
    for name, p in model_g.named_parameters():
        if p.grad is None or pc[name].grad is None or p.numel() < 4096:
            continue
        a, b = p.grad.float().cpu().flatten(), pc[name].grad.flatten()
        if b.norm() < 1e-8:
            continue
        cos = torch.dot(a, b) / (a.norm() * b.norm() + 1e-12)
        assert cos > 0.95, (name, cos.item())
        checked += 1
    assert checked > 10


def test_engine_step_with_gradient_sinks_matches_cpu():
    """Two optimizer steps through the training engine (flat buffers, weight gradients accumulated
    by the GEMM epilogue, fused AdamW) against the same engine on the CPU oracle path."""
    from wallx_b200.data.collator import to_device
    from wallx_b200.ops import gemm as G
    from wallx_b200.parallel.engine import TrainEngine

    cfg, model, batch = _build("flow")
    model_g = copy.deepcopy(model).to(torch.bfloat16).cuda()
    model_c = copy.deepcopy(model_g).float().cpu()
    gen = torch.Generator().manual_seed(2)
    extra = {"flow_noise": torch.randn(batch["action_chunk"].shape, generator=gen),
             "flow_time": torch.rand(batch["action_chunk"].shape[0], generator=gen) * 0.9}
    eng_g = TrainEngine(model_g, lr=1e-3, grad_accum=2)
    eng_c = TrainEngine(model_c, lr=1e-3, grad_accum=2)
    bg = to_device(batch, "cuda", torch.bfloat16)
    eg = {k: v.cuda() for k, v in extra.items()}
    for _ in range(2):
        for _mb in range(2):
            eng_c.backward(model_c(mode="train", **batch, **extra).loss)
            eng_g.backward(model_g(mode="train", **bg, **eg).loss)
        eng_c.optimizer_step(1e-3)
        eng_g.optimizer_step(1e-3)
    torch.cuda.synchronize()
    G.check_status()
    assert abs(eng_g.grad_norm().item() - eng_c.grad_norm().item()) / eng_c.grad_norm().item() < 0.05
    tot = agree = 0
    for bg_, bc_ in zip(eng_g.buffers, eng_c.buffers):
        s0, s1 = bc_.shard_range
        # the direction of the Adam update (sign of the first moment) agrees almost everywhere
        mg, mc = bg_.exp_avg[: bg_.numel].float().cpu(), bc_.exp_avg[: bc_.numel]
        big = mc.abs() > mc.abs().mean()
        tot += int(big.sum())
        agree += int((torch.sign(mg[big]) == torch.sign(mc[big])).sum())
    assert agree / max(tot, 1) > 0.97, agree / max(tot, 1)


def _predict_inputs(batch):
    drop = ("action_chunk", "labels", "pack_index", "seq_lens")
    return {k: v for k, v in batch.items() if k not in drop}


def test_flow_inference_gpu_matches_cpu_and_graph_matches_eager():
    """Prefix-KV flow sampler on the CUDA kernels: same chunk as the CPU fp32 oracle from the same
    noise, and the CUDA-graph Euler loop reproduces the eager loop."""
    from wallx_b200.data.collator import to_device
    from wallx_b200.ops import gemm as G

    cfg, model, batch = _build("flow")
    model_g = copy.deepcopy(model).to(torch.bfloat16).cuda().eval()
    model_c = copy.deepcopy(model_g).float().cpu().eval()
    inp = _predict_inputs(batch)
    B = inp["input_ids"].shape[0]
    A = model.action_preprocessor.action_dim
    noise = torch.randn(B, 16, A, generator=torch.Generator().manual_seed(3))
    out_c = model_c(mode="predict", predict_mode="diffusion", noise=noise, num_inference_timesteps=4, **inp)
    bg = to_device(inp, "cuda", torch.bfloat16)
    out_g = model_g(mode="predict", predict_mode="diffusion", noise=noise.cuda(), num_inference_timesteps=4, **bg)
    out_gg = model_g(mode="predict", predict_mode="diffusion", noise=noise.cuda(), num_inference_timesteps=4,
                     use_cuda_graph=True, **bg)
    torch.cuda.synchronize()
    G.check_status()
    a, b, c = out_c["predict_action"], out_g["predict_action"].cpu(), out_gg["predict_action"].cpu()
    assert a.shape == b.shape == (B, 16, A)
    scale = a.abs().max().item()
    assert (a - b).abs().max().item() < 0.08 * scale, ((a - b).abs().max().item(), scale)
    assert (b - c).abs().max().item() < 1e-3 * scale


def test_generate_gpu_matches_cpu():
    """Greedy decoding with the KV cache on the CUDA kernels vs the CPU oracle (tiny model)."""
    from wallx_b200.ops import gemm as G

    cfg, model, batch = _build("fast")
    model_g = copy.deepcopy(model).to(torch.bfloat16).cuda().eval()
    model_c = copy.deepcopy(model_g).float().cpu().eval()
    # prompt = everything up to a few tokens after the last image of sample 0
    ends = (batch["input_ids"][0] == cfg.vision_end_token_id).nonzero().flatten()
    n = int(ends.numel())
    ids = batch["input_ids"][:1, : int(ends[-1]) + 4]
    rows = int(batch["image_grid_thw"][:n].prod(1).sum())
    keep = {"pixel_values": batch["pixel_values"][:rows], "image_grid_thw": batch["image_grid_thw"][:n]}
    out_c = model_c.generate(input_ids=ids, max_new_tokens=6, **keep)
    kg = {k: (v.cuda().to(torch.bfloat16) if v.is_floating_point() else v.cuda()) for k, v in keep.items()}
    out_g = model_g.generate(input_ids=ids.cuda(), max_new_tokens=6, **kg)
    torch.cuda.synchronize()
    G.check_status()
    assert out_g.shape == out_c.shape
    # bf16 can flip a near-tie; the first generated token must agree and most of the rest
    new_c, new_g = out_c[0, ids.shape[1]:], out_g[0, ids.shape[1]:].cpu()
    assert new_c[0] == new_g[0]
    assert (new_c == new_g).float().mean() >= 0.5


def test_flow_engine_graph_matches_eager_sampler():
    """The serving engine (static buffers + one CUDA graph for ViT, prefix pass and Euler loop)
    returns the same chunk as ``predict`` for the same noise, also after the inputs change."""
    from wallx_b200.data.collator import to_device
    from wallx_b200.models.inference import FlowEngine
    from wallx_b200.ops import gemm as G

    cfg, model, batch = _build("flow")
    model_g = copy.deepcopy(model).to(torch.bfloat16).cuda().eval()
    inp = _predict_inputs(batch)
    B = inp["input_ids"].shape[0]
    A = model.action_preprocessor.action_dim
    gen = torch.Generator().manual_seed(7)
    eng = FlowEngine(model_g, inp, num_inference_timesteps=4)
    assert eng.graph is not None
    for trial in range(2):
        cur = dict(inp)
        if trial == 1:  # new observation, same layout
            cur["pixel_values"] = torch.randn(inp["pixel_values"].shape, generator=gen)
            cur["proprioception"] = torch.randn(inp["proprioception"].shape, generator=gen)
        noise = torch.randn(B, 16, A, generator=gen)
        ref = model_g(mode="predict", predict_mode="diffusion", noise=noise.cuda(), num_inference_timesteps=4,
                      **to_device(cur, "cuda", torch.bfloat16))["predict_action"]
        got = eng(cur, noise=noise)["predict_action"]
        torch.cuda.synchronize()
        scale = ref.abs().max().item()
        assert (ref - got).abs().max().item() < 1e-3 * scale
    G.check_status()


def test_training_is_bit_reproducible():
    """Two runs of the same two optimizer steps give bit-identical parameters (no float atomics on the
    training path: ordered column sums, norm-weight gradients and squared gradient norms)."""
    from wallx_b200.data.collator import to_device
    from wallx_b200.ops import gemm as G
    from wallx_b200.parallel.engine import TrainEngine

    def run():
        cfg, model, _ = _build("flow")
        from wallx_b200.data.collator import add_pack_info
        from wallx_b200.data.synthetic import make_batch

        m = copy.deepcopy(model).to(torch.bfloat16).cuda()
        eng = TrainEngine(m, lr=1e-3, weight_decay=0.1, max_grad_norm=1.0, grad_accum=1)
        g = torch.Generator().manual_seed(5)
        for _ in range(2):
            b = add_pack_info(make_batch(cfg, m.processor, 2, views=1, image_hw=(112, 112), prompt_len=16, horizon=16,
                                         generator=g), cfg)
            b["flow_noise"] = torch.randn(b["action_chunk"].shape, generator=g)
            b["flow_time"] = torch.rand(2, generator=g)
            eng.backward(m(mode="train", **to_device(b, "cuda", torch.bfloat16)).loss)
            eng.optimizer_step(1e-3)
        torch.cuda.synchronize()
        G.check_status()
        return {n: p.detach().clone() for n, p in m.named_parameters()}, eng.grad_norm().item()

    a, na = run()
    b, nb = run()
    assert na == nb
    for k in a:
        assert torch.equal(a[k], b[k]), k


@pytest.mark.parametrize("mode", ["flow", "fast"])
@pytest.mark.parametrize("with_engine", [False, True])
def test_fused_blocks_match_the_operator_path_bit_for_bit(mode, with_engine, monkeypatch):
    """One host call per decoder layer / vision block (csrc/blocks.cpp) launches the same kernels with the same
    arguments as the operator-by-operator path: loss and every gradient must be identical, with weight gradients
    returned to autograd (no engine) and with gradient sinks (engine)."""
    from wallx_b200.data.collator import to_device
    from wallx_b200.ops import blocks as BK
    from wallx_b200.ops import gemm as G
    from wallx_b200.parallel.engine import TrainEngine

    cfg, model, batch = _build(mode)
    extra = {}
    if mode == "flow":
        gen = torch.Generator().manual_seed(2)
        extra["flow_noise"] = torch.randn(batch["action_chunk"].shape, generator=gen).cuda()
        extra["flow_time"] = (torch.rand(batch["action_chunk"].shape[0], generator=gen) * 0.9).cuda()
    bg = to_device(batch, "cuda", torch.bfloat16)
    results = []
    for fused in (False, True):
        monkeypatch.setattr(BK, "ENABLED", fused)
        m = copy.deepcopy(model).to(torch.bfloat16).cuda()
        eng = TrainEngine(m, lr=1e-3, grad_accum=1) if with_engine else None
        out = m(mode="train", **bg, **extra)
        out.loss.backward()
        torch.cuda.synchronize()
        G.check_status()
        grads = {n: p.grad.detach().clone() for n, p in m.named_parameters() if p.grad is not None}
        if eng is not None:
            eng.optimizer_step(1e-3)
            grads.update({"param:" + n: p.detach().clone() for n, p in m.named_parameters()})
            eng.close()
        results.append((out.loss.detach().clone(), grads))
    (l0, g0), (l1, g1) = results
    assert torch.equal(l0, l1)
    assert set(g0) == set(g1) and len(g0) > 20
    for n in g0:
        assert torch.equal(g0[n], g1[n]), n

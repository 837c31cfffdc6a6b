"""Numerical parity with the reference's own classes (skipped when the reference is not installed under
``baseline/_ref``): the reference's ``Qwen2_5_VLMoEForAction`` is built at the tiny configuration, its ``state_dict()``
is loaded into this framework's model by the checkpoint key names, and both run the same batch.

The reference's flash-attention path is causal over all tokens and uses the section layout of its CUDA mRoPE kernel
(modeling_qwen2_5_vl_act.py:557-558, fusions/ops.py:451), i.e. ``action_attn="causal"`` and
``mrope_layout="wallx_cuda"`` here. Both models compute in bf16 with different kernels and different summation orders
(cuBLAS + flash-attn 2 there, tcgen05 kernels here), so the tolerances are those of bf16 forward passes: 3 % on
losses, 0.99 cosine on logits and predicted actions.
"""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def _reference_model(cfg, dev, fast):
    from wallx_b200.bench import ref_shims

    ref_shims.install(REF_DIR)
    from wall_x.model.qwen2_5_based.configuration_qwen2_5_vl import Qwen2_5_VLConfig as RefConfig  # reference
    from wall_x.model.qwen2_5_based.modeling_qwen2_5_vl_act import Qwen2_5_VLMoEForAction as RefModel  # reference

    from wallx_b200.data.synthetic import make_processor

    d = cfg.to_dict()
    for k in ("architectures", "model_type", "mrope_layout", "action_attn", "output_attentions", "output_hidden_states",
              "use_return_dict"):
        d.pop(k, None)
    d["vision_config"]["initializer_range"] = 0.02
    rcfg = RefConfig(**d)
    rcfg._attn_implementation = "flash_attention_2"
    rcfg.vision_config._attn_implementation = "flash_attention_2"
    proc = make_processor(cfg, 16)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = RefModel(rcfg, use_fast_tokenizer=fast, processor=proc)
    finally:
        torch.set_default_dtype(old)
    return model.to(torch.bfloat16), proc


def _restore_alias_package():
    """The shim puts the reference's ``wall_x`` first on the path; later tests expect this repository's alias package."""
    for k in [k for k in sys.modules if k == "wall_x" or k.startswith("wall_x.")]:
        del sys.modules[k]
    while REF_DIR in sys.path:
        sys.path.remove(REF_DIR)


def _stage(batch, dev):
    out = {}
    for k, v in batch.items():
        if isinstance(v, torch.Tensor):
            v = v.to(dev)
            if v.is_floating_point():
                v = v.to(torch.bfloat16)
        out[k] = v
    return out


def _cos(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))


@pytest.mark.timeout(900)
@pytest.mark.parametrize("mode", ["flow", "fast"])
def test_same_weights_give_the_same_losses_logits_and_actions(mode):
    if not os.path.isdir(os.path.join(REF_DIR, "wall_x")):
        pytest.skip("reference not installed under baseline/_ref")
    from wallx_b200.config import tiny_config
    from wallx_b200.data.collator import add_pack_info
    from wallx_b200.data.synthetic import make_batch
    from wallx_b200.models import Qwen2_5_VLMoEForAction
    from wallx_b200.ops import gemm as G

    dev = torch.device("cuda", 0)
    cfg = tiny_config(mrope_layout="wallx_cuda", action_attn="causal")
    try:
        torch.manual_seed(0)
        ref, proc = _reference_model(cfg, dev, fast=(mode == "fast"))
        with torch.no_grad():  # the reference's constructor leaves most weights at their defaults: randomise all of them
            gen = torch.Generator(device="cuda").manual_seed(3)
            for n, p in ref.named_parameters():
                if p.dim() >= 2:
                    p.copy_(torch.randn(p.shape, device=dev, generator=gen) * 0.05)
                elif "norm" in n or "ln_q" in n:
                    p.copy_(1.0 + 0.1 * torch.randn(p.shape, device=dev, generator=gen))
                elif "normalizer" not in n:
                    p.copy_(0.02 * torch.randn(p.shape, device=dev, generator=gen))
        ours = Qwen2_5_VLMoEForAction(cfg, processor=proc, use_fast_tokenizer=(mode == "fast")).to(torch.bfloat16).to(dev)
        missing, unexpected = ours.load_state_dict(ref.state_dict(), strict=False)
        assert not [k for k in unexpected if "inv_freq" not in k and "rotary" not in k], unexpected
        assert not [k for k in missing if "inv_freq" not in k], missing
        g = torch.Generator().manual_seed(11)
        batch = make_batch(cfg, proc, 3, views=2, image_hw=(112, 112), prompt_len=16, horizon=16, mode=mode, fast_tokens=12,
                           generator=g)
        rb = _stage(batch, dev)
        ob = _stage(add_pack_info(dict(batch), cfg), dev)

        # ---- training forward: the reference draws its noise and time from the global CUDA generator, first thing
        extra = {}
        if mode == "flow":
            a = rb["action_chunk"]
            torch.manual_seed(21)
            noise = torch.randn_like(a)
            time = ref.action_preprocessor.sample_time(a.shape[0], a.device, a.dtype)
            extra = {"flow_noise": noise, "flow_time": time}
            torch.manual_seed(21)
        ref.train()
        ours.train()
        with torch.no_grad():
            r_out = ref(**rb, mode="train")
            o_out = ours(mode="train", **ob, **extra)
        torch.cuda.synchronize()
        G.check_status()
        rl, ol = float(r_out.loss), float(o_out.loss)
        assert abs(rl - ol) / max(abs(rl), 1e-3) < 0.03, (mode, rl, ol)
        if mode == "flow":
            assert abs(float(r_out.flow_loss) - float(o_out.flow_loss)) / max(float(r_out.flow_loss), 1e-3) < 0.03
        else:
            assert abs(float(r_out.cross_entropy_loss) - float(o_out.cross_entropy_loss)) / float(r_out.cross_entropy_loss) < 0.03

        # ---- logits of every position (validate mode)
        ref.eval()
        ours.eval()
        vb = {k: v for k, v in rb.items() if k not in ("action_chunk",)} if mode == "fast" else rb
        if mode == "fast":
            with torch.no_grad():
                r_log = ref(**vb, mode="validate").logits
                o_log = ours(mode="validate", return_logits=True, **{k: v for k, v in ob.items() if k != "action_chunk"}).logits
            mask = rb["attention_mask"].bool()
            assert r_log.shape == o_log.shape, (r_log.shape, o_log.shape)
            assert _cos(r_log[mask], o_log[mask]) > 0.99
            agree = (r_log[mask].argmax(-1) == o_log[mask].argmax(-1)).float().mean()
            assert agree > 0.9, float(agree)

        # ---- flow-matching inference from the same initial noise: the reference integrates linspace(0, 1, n) with
        # n - 1 Euler evaluations and re-runs the whole sequence each time; here the prefix is cached
        if mode == "flow":
            inp = {k: v for k, v in rb.items() if k not in ("action_chunk", "labels")}
            oin = {k: v for k, v in ob.items() if k not in ("action_chunk", "labels")}
            H, A = rb["action_chunk"].shape[1], rb["action_chunk"].shape[2]
            torch.manual_seed(33)
            x0 = torch.randn((rb["input_ids"].shape[0], H, A), dtype=torch.bfloat16, device=dev)
            torch.manual_seed(33)
            with torch.no_grad():
                r_act = ref(**inp, mode="predict", predict_mode="diffusion", num_inference_timesteps=6, pred_horizon=H,
                            action_dim=A)["predict_action"]
                o_act = ours(mode="predict", predict_mode="diffusion", num_inference_timesteps=6, reference_grid=True,
                             noise=x0, **oin)["predict_action"]
            torch.cuda.synchronize()
            G.check_status()
            assert r_act.shape == o_act.shape
            assert _cos(r_act, o_act) > 0.99, _cos(r_act, o_act)
            assert float((r_act.float() - o_act.float()).abs().max()) < 0.1 * float(r_act.float().abs().max()) + 0.05
    finally:
        _restore_alias_package()

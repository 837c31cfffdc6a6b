"""The reference's import paths resolve to this framework (drop-in for user code)."""
import torch


def test_reference_module_paths_resolve():
    from wall_x.data.config import ACTION_DATASET_NAMES, X2RDataProcessingConfig  # noqa: F401
    from wall_x.data.load_lerobot_dataset import DataCollator, PreprocessedDataset, get_data_configs, load_test_dataset  # noqa: F401
    from wall_x.data.utils import get_wallx_normal_text, preprocesser_call, replace_action_token  # noqa: F401
    from wall_x.model.action_head import ActionProcessor, Normalizer  # noqa: F401
    from wall_x.model.qwen2_5_based.configuration_qwen2_5_vl import Qwen2_5_VLConfig
    from wall_x.model.qwen2_5_based.modeling_qwen2_5_vl_act import Qwen2_5_VLMoEForAction
    from wall_x.trainer.qwen_vl_act_trainer import QwenVlAct_Trainer  # noqa: F401
    from wall_x.utils.constant import action_statistic_dof
    from wall_x.utils.timers import Timers  # noqa: F401

    import wallx_b200.config as C
    import wallx_b200.models as M

    assert Qwen2_5_VLMoEForAction is M.Qwen2_5_VLMoEForAction
    assert Qwen2_5_VLConfig is C.Qwen2_5_VLConfig
    assert len(action_statistic_dof) >= 27 and "x2_normal" in action_statistic_dof


def test_reference_named_ops_exist_and_run_on_cpu():
    from wall_x.fusions import ops

    for name in ("permute", "unpermute", "get_rope_index", "rot_pos_emb", "get_window_index"):
        assert hasattr(ops, name), name
    x = torch.randn(10, 8)
    idx = torch.tensor([1, 0, 0, 1, 1, 0, 0, 0, 1, 0], dtype=torch.int32)
    permuted, row_map = ops.permute(x, idx)
    back = ops.unpermute(permuted, row_map)
    assert torch.allclose(back, x)
    # tokens of expert 0 come first, in their original order (stable)
    assert torch.equal(permuted[:6], x[idx == 0])


def test_plain_qwen2_5_vl_trains_and_generates():
    """The non-MoE base model: one FFN per layer, Hugging Face key names, text loss and greedy decoding."""
    from wall_x.model.qwen2_5_based.modeling_qwen2_5_vl import Qwen2_5_VLForConditionalGeneration, Qwen2_5_VLModel

    from wallx_b200.config import tiny_config
    from wallx_b200.data.synthetic import make_batch, make_processor

    cfg = tiny_config()
    proc = make_processor(cfg, 16)
    torch.manual_seed(0)
    m = Qwen2_5_VLForConditionalGeneration(cfg, processor=proc, use_fast_tokenizer=True).float()
    assert m.model.layers[0].moe is None
    keys = set(m.state_dict())
    assert "model.layers.0.mlp.gate_proj.weight" in keys and "model.layers.1.mlp.down_proj.weight" in keys
    assert not any(".moe." in k for k in keys)
    b = make_batch(cfg, proc, 2, views=1, image_hw=(112, 112), prompt_len=16, horizon=8, mode="fast", fast_tokens=6,
                   generator=torch.Generator().manual_seed(1))
    out = m(mode="train", **b)
    out.loss.backward()
    assert torch.isfinite(out.loss) and m.model.layers[0].mlp.gate_up_weight.grad.abs().sum() > 0
    ids = b["input_ids"][:1, :30]
    gen = m.generate(input_ids=ids, max_new_tokens=3, pixel_values=b["pixel_values"][:64], image_grid_thw=b["image_grid_thw"][:1])
    assert gen.shape == (1, 33)
    core = Qwen2_5_VLModel(tiny_config())
    assert core.layers[0].mlp is not None and core.layers[0].moe is None

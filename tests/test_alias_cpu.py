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


# every top-level class / function / table of the reference's Python modules, by module path
_REFERENCE_NAMES = {
    "wall_x.data.load_lerobot_dataset": "CAMERA_KEY_MAPPINGS PreprocessedDataset DataCollator load_lerobot_data "
                                        "get_distributed_dataloader get_data_configs TestDataset load_test_dataset",
    "wall_x.data.utils": "CAMERA_NAME_MAPPING MULTIMODAL_DATASET_NAMES FREQUENCY_MAPPING preprocesser_call "
                         "process_grounding_points get_frame_instruction get_task_instruction get_wallx_normal_text "
                         "get_action_tokens pad_action_token_strs replace_action_token",
    "wall_x.data.config": "TACTILE_FILE_MAPPING ACTION_DATASET_NAMES MULTIMODAL_DATASET_NAMES X2RDataProcessingConfig",
    "wall_x.trainer.qwen_vl_act_trainer": "timer print_rank_last seed_all QwenVlAct_Trainer",
    "wall_x.model.action_head": "Normalizer SinusoidalPosEmb ActionProcessor",
    "wall_x.utils.timers": "TimerBase DummyTimer Timer Timers",
    "wall_x.utils.constant": "action_statistic_dof",
    "wall_x.fusions.ops": "AsymmetricDualExpertGemm asym_dual_gmm PermuteMoE_topK UnpermuteMoE_topK permute unpermute "
                          "MultimodalRoPE multimodal_rope get_rope_index rot_pos_emb get_window_index",
    "wall_x.fusions.backend": "asym_dual_gmm_separated permute unpermute unpermute_bwd rope rope_bwd get_rope_index "
                              "rot_pos_emb get_window_index",
    "wall_x.model.qwen2_5_based.configuration_qwen2_5_vl": "Qwen2_5_VLVisionConfig Qwen2_5_VLConfig",
    "wall_x.model.qwen2_5_based.modeling_qwen2_5_vl_act": "Qwen2_5_VLACausalLMOutputWithPast BlockSparseMLP SparseMoeBlock "
                                                          "QWEN2_5_VL_ATTENTION_CLASSES Qwen2_5_VLDecoderLayer_with_MoE "
                                                          "Qwen2_5_VLMoEModel Qwen2_5_VLMoEForAction",
    "wall_x.model.qwen2_5_based.modeling_qwen2_5_vl": "Qwen2_5_VLMLP Qwen2_5_VisionPatchEmbed Qwen2_5_VisionRotaryEmbedding "
        "Qwen2RMSNorm Qwen2_5_VLPatchMerger apply_rotary_pos_emb_flashatt Qwen2_5_VLVisionFlashAttention2 rotate_half "
        "apply_rotary_pos_emb_vision Qwen2_5_VLVisionAttention Qwen2_5_VLVisionSdpaAttention "
        "QWEN2_5_VL_VISION_ATTENTION_CLASSES Qwen2_5_VLVisionBlock Qwen2_5_VLPreTrainedModel "
        "Qwen2_5_VisionTransformerPretrainedModel Qwen2_5_VLRotaryEmbedding Qwen2MLP apply_multimodal_rotary_pos_emb "
        "repeat_kv Qwen2_5_VLAttention Qwen2_5_VLFlashAttention2 Qwen2_5_VLSdpaAttention QWEN2_5_VL_ATTENTION_CLASSES "
        "Qwen2_5_VLDecoderLayer Qwen2_5_VLModel Qwen2_5_VLCausalLMOutputWithPast Qwen2_5_VLForConditionalGeneration",
}


def test_every_public_name_of_the_reference_modules_resolves():
    import importlib

    missing = []
    for mod, names in _REFERENCE_NAMES.items():
        m = importlib.import_module(mod)
        missing += [f"{mod}.{n}" for n in names.split() if not hasattr(m, n)]
    assert not missing, missing


def test_rotary_building_blocks_match_the_oracle():
    from wall_x.model.qwen2_5_based import modeling_qwen2_5_vl as VL
    from wallx_b200.config import tiny_config
    from wallx_b200.ops import ref

    torch.manual_seed(0)
    cfg = tiny_config()
    D = cfg.head_dim
    sections = list(cfg.rope_scaling["mrope_section"])
    rot = VL.Qwen2_5_VLRotaryEmbedding(cfg)
    B, S, H = 2, 7, 3
    pos = torch.randint(0, 50, (3, B, S))
    x = torch.randn(B, H, S, D)
    cos, sin = rot(x, pos)
    assert cos.shape == (3, B, S, D)
    q, k = torch.randn(B, H, S, D), torch.randn(B, 1, S, D)
    qo, ko = VL.apply_multimodal_rotary_pos_emb(q, k, cos, sin, sections)
    for b in range(B):
        c, s = ref.mrope_cos_sin(pos[:, b], ref.rope_inv_freq(D, cfg.rope_theta), sections, "hf")
        want = ref.apply_rope(q[b].transpose(0, 1), c, s).transpose(0, 1)
        assert torch.allclose(qo[b], want, atol=1e-5)
    assert torch.allclose(ko.norm(dim=-1), k.norm(dim=-1), atol=1e-5)  # a rotation
    # vision tower
    vr = VL.Qwen2_5_VisionRotaryEmbedding(8)
    tab = vr(5)
    assert tab.shape == (5, 4) and torch.allclose(tab[3], 3 * vr.inv_freq)
    emb = torch.cat([tab, tab], dim=-1)
    qv, kv = torch.randn(5, 2, 8), torch.randn(5, 2, 8)
    a, b_ = VL.apply_rotary_pos_emb_vision(qv, kv, emb.cos(), emb.sin())
    assert torch.allclose(a, ref.apply_rope(qv, emb.cos(), emb.sin()), atol=1e-6)
    a2, _ = VL.apply_rotary_pos_emb_flashatt(qv, kv, emb.cos(), emb.sin())
    assert torch.equal(a, a2)
    r = VL.repeat_kv(k, 3)
    assert r.shape == (B, 3, S, D) and torch.equal(r[:, 0], r[:, 2]) and torch.equal(r[:, 1], k[:, 0])
    assert VL.QWEN2_5_VL_ATTENTION_CLASSES["sdpa"] is VL.Qwen2_5_VLFlashAttention2
    # timers keep their base class
    from wall_x.utils.timers import DummyTimer, Timer, TimerBase

    assert issubclass(Timer, TimerBase) and issubclass(DummyTimer, TimerBase)
    t = Timer("x", use_cuda_events=False)
    t.start()
    t.stop()
    assert t.elapsed() >= 0.0

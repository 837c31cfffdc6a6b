"""Data path on CPU: prompt template, labels, FAST substitution, collator, dataset wrapper."""
import numpy as np
import torch

from wallx_b200.config import tiny_config
from wallx_b200.data import text as T
from wallx_b200.data.collator import DataCollator, minmax_normalize
from wallx_b200.data.lerobot import PreprocessedDataset, SyntheticEpisodeDataset, get_data_configs
from wallx_b200.data.synthetic import images_to_patches, make_processor, smart_resize


def test_prompt_template_exact():
    txt, sub = T.get_wallx_normal_text({"instruction": "open the drawer"}, 3, 0, None,
                                       {"k1": "face_view", "k2": "move1_view"})
    assert not sub
    assert txt == ("<|im_start|>system\nYou are a helpful assistant.<|im_end|>\n<|im_start|>user\nObservation: "
                   "front view: <|vision_start|><|image_pad|><|vision_end|> move view: <|vision_start|><|image_pad|>"
                   "<|vision_end|>\nInstruction: open the drawer\nPredict the next action in robot action.\n"
                   "Proprioception: <|propri|>\n<|im_end|>\n<|im_start|>assistant\n<|action_fast|><|im_end|>\n"
                   "<|action|><|action|><|action|>")
    flow = T.replace_action_token([txt], None, None, ["x2_normal"])[0]
    assert "<|action_fast|>" not in flow and flow.endswith("<|im_start|>assistant\n" + "<|action|>" * 3)


def test_frame_instruction_and_priority():
    info = {"instruction": "base", "subtask_generation": {"0 10": "first", "10 20": "second"}}
    got, end = T.get_frame_instruction(info, frame_idx=12)
    assert got == {"instruction": "base", "subtask_generation": "second"} and end == 21
    assert T.get_task_instruction(got) == "\nsecond"
    assert T.get_task_instruction({"instruction": "only"}) == "only"


def test_grounding_points():
    s = T.process_grounding_points("a <point>[100, 50]</point> b <point>[0, 0, 199, 99]</point>", 100, 200, 50, 100, "qwen2_5")
    assert s == "a <point>[50, 25]</point> b <point>[0, 0, 99, 49]</point>"
    s2 = T.process_grounding_points("<point>[100, 50]</point>", 100, 200, 50, 100, "qwen2")
    assert s2 == "<point>[500.0, 500.0]</point>"


def test_fast_substitution_and_labels():
    cfg = tiny_config()
    proc = make_processor(cfg, 16)

    class FakeFast:
        vocab_size = 16

        def __call__(self, arr):
            return [[int(abs(v) * 7) % 16 for v in np.asarray(arr).reshape(-1)[:5]]]

    txt, _ = T.get_wallx_normal_text({"instruction": "go"}, 4, 0, None, {"a": "face_view"})
    act = torch.rand(1, 32, 20) * 2 - 1
    mask = torch.ones(1, 32, 20)
    out = T.replace_action_token([txt], act, FakeFast(), ["x2_normal"], mask)[0]
    assert "<|action|>" not in out and "<|action_fast|>" not in out and out.count("<|action_token_") == 5
    imgs = [np.zeros((56, 56, 3), dtype=np.uint8)]
    enc = T.preprocesser_call(proc, images=imgs, text=[out], padding=True)
    labels, ids = enc["labels"], enc["input_ids"]
    tok = proc.tokenizer
    learn = ids[labels != -100].tolist()
    assert len(learn) == 5 + 2 and all(t >= tok.action_start for t in learn[:5])
    assert learn[5] == tok.convert_tokens_to_ids("<|im_end|>")
    n_img = (ids == cfg.image_token_id).sum().item()
    assert n_img == 4  # 56 px -> 4x4 patches -> 2x2 merged tokens


def test_smart_resize_and_patch_layout():
    assert smart_resize(256, 256) == (252, 252) and smart_resize(112, 112) == (112, 112)
    img = torch.arange(56 * 56 * 3, dtype=torch.float32).reshape(1, 56, 56, 3).remainder(251).to(torch.uint8)
    pv, grid = images_to_patches(img)
    assert grid == [[1, 4, 4]] and pv.shape == (16, 1176)
    # patch 0 = rows 0..13, cols 0..13; channel-major, the frame repeated twice along time
    x = img[0].permute(2, 0, 1).float() / 255.0
    mean = torch.tensor([0.48145466, 0.4578275, 0.40821073]).view(3, 1, 1)
    std = torch.tensor([0.26862954, 0.26130258, 0.27577711]).view(3, 1, 1)
    x = (x - mean) / std
    p0 = x[:, :14, :14].unsqueeze(1).expand(3, 2, 14, 14).reshape(-1)
    assert torch.allclose(pv[0], p0, atol=1e-6)
    # patches come in 2x2 merge blocks: index 3 is patch (row 1, col 1), index 4 is patch (row 0, col 2)
    p3 = x[:, 14:28, 14:28].unsqueeze(1).expand(3, 2, 14, 14).reshape(-1)
    assert torch.allclose(pv[3], p3, atol=1e-6)
    p4 = x[:, :14, 28:42].unsqueeze(1).expand(3, 2, 14, 14).reshape(-1)
    assert torch.allclose(pv[4], p4, atol=1e-6)


def test_collator_and_dataset_end_to_end():
    cfg = tiny_config()
    proc = make_processor(cfg, 16)
    conf = {"batch_size_per_gpu": 3, "num_workers": 0,
            "data": {"action_horizon": 16, "resolution": {"face_view": 112, "left_wrist_view": 112, "right_wrist_view": 112}}}
    dc = get_data_configs(conf["data"])
    assert dc["action_horizon"] == 17
    ds = SyntheticEpisodeDataset(n=40, horizon=16)
    ds.actions[0, 0, 0] = float("nan")
    pre = PreprocessedDataset(ds, conf, dc, processor=proc, model_config=cfg)
    assert len(pre.train_dataset) == 38 and len(pre.val_dataset) == 2
    loader, sampler = pre.get_train_dataloader()
    batch = next(iter(loader))
    B, S = batch["input_ids"].shape
    assert B == 3 and batch["action_chunk"].shape == (3, 16, 20) and batch["proprioception"].shape == (3, 1, 20)
    assert batch["dof_mask"][..., 14:].sum() == 0 and batch["action_chunk"].abs().max() <= 1.0
    assert (batch["moe_token_types"].sum(1) == 16).all() and "labels" not in batch
    assert batch["pixel_values"].shape[1] == 1176 and batch["image_grid_thw"].shape == (9, 3)
    assert batch["position_ids"].shape == (3, B, S) and batch["pack_index"].numel() == batch["attention_mask"].sum()
    col = DataCollator(conf, dc, ds.meta.stats, processor=proc)
    item = pre[0]
    item["action"] = item["action"].clone()
    item["action"][0, 0] = float("nan")
    b2 = col([item])
    assert b2["dof_mask"][0, 0, 0] == 0 and b2["action_chunk"][0, 0, 0] == minmax_normalize(torch.zeros(1), [-3.0], [3.0])


def test_distributed_dataloader_helper_shards_without_overlap():
    """``get_distributed_dataloader`` (the reference's helper name): two ranks see disjoint halves of the training
    split, the validation loader is not shuffled."""
    from wall_x.data.load_lerobot_dataset import get_distributed_dataloader

    cfg = tiny_config()
    proc = make_processor(cfg, 16)
    conf = {"batch_size_per_gpu": 2, "num_workers": 0,
            "data": {"action_horizon": 16, "resolution": {"face_view": 112, "left_wrist_view": 112, "right_wrist_view": 112}}}
    dc = get_data_configs(conf["data"])
    pre = PreprocessedDataset(SyntheticEpisodeDataset(n=40, horizon=16), conf, dc, processor=proc, model_config=cfg)
    seen = []
    for rank in range(2):
        loader, sampler = get_distributed_dataloader(pre, conf, rank=rank, world_size=2, seed=7, is_train=True)
        sampler.set_epoch(0)
        seen.append(list(iter(sampler)))
        assert len(loader) == len(seen[-1]) // 2
    assert not set(seen[0]) & set(seen[1]) and len(seen[0]) == len(seen[1]) == 19
    vloader, vsampler = get_distributed_dataloader(pre, conf, rank=0, world_size=1, is_train=False)
    assert list(iter(vsampler)) == list(range(len(vsampler)))
    batch = next(iter(vloader))
    assert batch["input_ids"].shape[0] <= 2

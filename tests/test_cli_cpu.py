"""Command-line tools and the built-in FAST-style tokenizer on CPU with the synthetic model."""
import os

import numpy as np
import torch

from wallx_b200.cli import draw_openloop_plot, fake_inference, merge_tokenizer, vqa_inference
from wallx_b200.data.fast_tokenizer import DctActionTokenizer


def test_dct_action_tokenizer_round_trip():
    tok = DctActionTokenizer(2048)
    rng = np.random.default_rng(0)
    smooth = np.cumsum(rng.normal(size=(2, 32, 14)) * 0.03, axis=1).clip(-1, 1)
    ids = tok(smooth)
    assert len(ids) == 2 and all(0 <= i < 2048 for row in ids for i in row)
    assert len(ids[0]) < 32 * 14  # trailing zero coefficients are dropped
    back = tok.decode(ids, time_horizon=32, action_dim=14)
    assert back.shape == (2, 32, 14) and np.abs(back - smooth).max() < 0.1
    # undecodable input -> all-zero chunk (callers treat that as "no prediction")
    assert tok.decode([[5000]], 32, 14).sum() == 0 and tok.decode([[]], 32, 14).sum() == 0
    assert tok(torch.zeros(32, 14))[0] == [tok.zero]


def test_fake_inference_synthetic():
    assert fake_inference.main(["--synthetic", "--device", "cpu", "--seq-length", "24"]) == 0


def test_merge_tokenizer_synthetic(tmp_path):
    assert merge_tokenizer.main(["--synthetic", "16", "--out", str(tmp_path / "tok")]) == 0
    import json

    d = json.load(open(tmp_path / "tok" / "synthetic_tokenizer.json"))
    assert d["init_kwargs"] == {"action_token_vocab_size": 16, "action_token_start_index": 1002}
    assert d["special"]["<|propri|>"] == 1000 and d["special"]["<|action|>"] == 1001 and d["length"] == 1018


def test_vqa_wrapper_synthetic():
    w = vqa_inference.VQAWrapper(synthetic=True, device="cpu")
    img = torch.randint(0, 256, (56, 56, 3), dtype=torch.uint8)
    ans = w.generate(img, "what is in the image?", max_new_tokens=4)
    assert isinstance(ans, str) and len(ans) > 0


def test_openloop_plot_synthetic(tmp_path):
    for mode in ("diffusion", "fast"):
        out = tmp_path / mode
        rc = draw_openloop_plot.main(["--synthetic", "--device", "cpu", "--save-dir", str(out), "--pred-horizon", "8",
                                      "--frames", "20", "--predict-mode", mode])
        assert rc == 0
        assert os.path.exists(out / "lerobot_comparison.csv")
        assert os.path.exists(out / "lerobot_comparison.svg") or os.path.exists(out / "lerobot_comparison.png")
        rows = open(out / "lerobot_comparison.csv").read().strip().split("\n")
        assert len(rows) == 21

"""Random-input smoke test of a checkpoint: one ``mode="validate"`` forward, then shape / NaN / Inf
checks on the logits (reference: scripts/fake_inference.py:1-85).

``python -m wallx_b200.cli.fake_inference --model /path/to/model`` or ``--synthetic``.
"""
from __future__ import annotations

import argparse
import sys

import torch

from ._common import load_model, pick_device


def run(model, batch_size: int = 1, seq_length: int = 50, seed: int = 0):
    dev = model.device
    float_dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    g = torch.Generator().manual_seed(seed)
    vocab = len(model.processor.tokenizer) if getattr(model, "processor", None) is not None else model.config.vocab_size
    cfg = model.config
    ids = torch.randint(0, vocab, (batch_size, seq_length), generator=g)
    # random ids must not contain placeholders that would demand pixel inputs
    for special in (cfg.image_token_id, cfg.video_token_id):
        ids[ids == special] = 0
    P = sum(cfg.agent_pos_config.values()) if getattr(cfg, "agent_pos_config", None) else 20
    A = sum(cfg.dof_config.values())
    batch = dict(
        input_ids=ids.to(dev),
        attention_mask=torch.ones(batch_size, seq_length, dtype=torch.long, device=dev),
        moe_token_types=torch.zeros(batch_size, seq_length, dtype=torch.long, device=dev),
        position_ids=torch.arange(seq_length).unsqueeze(0).expand(batch_size, -1).to(dev),
        proprioception=torch.randn(batch_size, 1, P, generator=g).to(dev, float_dtype),
        agent_pos_mask=torch.ones(batch_size, 1, P).to(dev, float_dtype),
        dof_mask=torch.ones(batch_size, 32, A).to(dev, float_dtype),
        dataset_names=["x2_normal"] * batch_size,
    )
    with torch.no_grad():
        out = model(mode="validate", **batch)
    logits = out.logits
    report = {
        "shape": tuple(logits.shape),
        "shape_ok": tuple(logits.shape) == (batch_size, seq_length, model.model.embed_tokens.weight.shape[0]),
        "nan": bool(torch.isnan(logits).any()),
        "inf": bool(torch.isinf(logits).any()),
        "min": float(logits.float().min()), "max": float(logits.float().max()),
        "mean": float(logits.float().mean()), "std": float(logits.float().std()),
    }
    return report


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--seq-length", type=int, default=50)
    args = ap.parse_args(argv)
    model = load_model(args.model, args.synthetic, pick_device(args.device))
    rep = run(model, args.batch_size, args.seq_length)
    ok = rep["shape_ok"] and not rep["nan"] and not rep["inf"]
    print("fake inference:", "ok" if ok else "FAILED")
    for k, v in rep.items():
        print(f"  {k}: {v}")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())

"""Open-loop evaluation plot: predicted vs ground-truth actions over one episode
(reference: scripts/draw_openloop_plot.py:1-86).

Every ``pred_horizon``-th frame the model predicts a whole action chunk (``--predict-mode fast`` as in
the reference, or ``diffusion``); predictions and de-normalised ground truth are written to
``<save-dir>/lerobot_comparison.csv`` and plotted per action dimension to
``lerobot_comparison.png`` (matplotlib, when installed) or ``lerobot_comparison.svg`` (built-in
writer). ``--synthetic`` uses a tiny random model and a synthetic episode dataset.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

from ._common import load_model, pick_device


def rollout(model, dataloader, pred_horizon: int, action_dim: int, predict_mode: str, dataset_name: str = "x2_normal"):
    dev = model.device
    float_dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    total = len(dataloader)
    gt = torch.zeros(total, action_dim)
    pred = torch.zeros(total, action_dim)
    for idx, batch in enumerate(dataloader):
        if idx % pred_horizon != 0 or idx + pred_horizon >= total:
            continue
        b = {k: (v.to(dev, float_dtype) if torch.is_tensor(v) and v.is_floating_point()
                 else (v.to(dev) if torch.is_tensor(v) else v)) for k, v in dict(batch).items()}
        # the flow sampler integrates over the model's full (padded) action width; FAST decoding
        # reshapes the decoded tokens to the requested width
        ad = model.action_preprocessor.action_dim if predict_mode == "diffusion" else action_dim
        with torch.no_grad():
            out = model(**b, action_dim=ad, pred_horizon=pred_horizon, mode="predict", predict_mode=predict_mode)
        pa = out["predict_action"]
        if pa is not None:
            pa = pa.detach().float().cpu().reshape(-1, pa.shape[-1])[:pred_horizon, :action_dim]
            pred[idx:idx + pa.shape[0], : pa.shape[1]] = pa
        chunk = b["action_chunk"][:, :pred_horizon, :action_dim]
        dof = b["dof_mask"][:, :pred_horizon, :].to(chunk.dtype)
        g = model.action_preprocessor.normalizer_action.unnormalize_data(chunk.float(), [dataset_name], dof.float())
        g = g.detach().cpu().reshape(-1, g.shape[-1])[:, :action_dim]
        gt[idx:idx + g.shape[0]] = g
    return gt, pred


def write_csv(path, gt, pred):
    with open(path, "w") as f:
        d = gt.shape[1]
        f.write("t," + ",".join(f"gt_{i}" for i in range(d)) + "," + ",".join(f"pred_{i}" for i in range(d)) + "\n")
        for t in range(gt.shape[0]):
            f.write(f"{t}," + ",".join(f"{v:.6f}" for v in gt[t].tolist()) + "," +
                    ",".join(f"{v:.6f}" for v in pred[t].tolist()) + "\n")


def write_svg(path, gt, pred, title="Action Comparison for lerobot"):
    """One panel per action dimension, ground truth (blue) and prediction (orange)."""
    T, D = gt.shape
    W, H, pad = 900, 160, 40
    parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{D * H + 40}" font-family="sans-serif" font-size="11">',
             f'<text x="{W // 2}" y="18" text-anchor="middle" font-size="15">{title}</text>']
    for i in range(D):
        y0 = 30 + i * H
        lo = min(float(gt[:, i].min()), float(pred[:, i].min()))
        hi = max(float(gt[:, i].max()), float(pred[:, i].max()))
        span = (hi - lo) or 1.0

        def pts(series):
            return " ".join(f"{pad + (W - 2 * pad) * t / max(T - 1, 1):.1f},{y0 + (H - 30) * (1 - (float(v) - lo) / span):.1f}"
                            for t, v in enumerate(series.tolist()))

        parts.append(f'<rect x="{pad}" y="{y0}" width="{W - 2 * pad}" height="{H - 30}" fill="none" stroke="#999"/>')
        parts.append(f'<polyline fill="none" stroke="#1f77b4" points="{pts(gt[:, i])}"/>')
        parts.append(f'<polyline fill="none" stroke="#ff7f0e" points="{pts(pred[:, i])}"/>')
        parts.append(f'<text x="4" y="{y0 + 12}">dim {i + 1}</text>')
    parts.append("</svg>")
    with open(path, "w") as f:
        f.write("\n".join(parts))


def plot(save_dir, gt, pred):
    os.makedirs(save_dir, exist_ok=True)
    write_csv(os.path.join(save_dir, "lerobot_comparison.csv"), gt, pred)
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        out = os.path.join(save_dir, "lerobot_comparison.svg")
        write_svg(out, gt, pred)
        return out
    D = gt.shape[1]
    fig, axs = plt.subplots(D, 1, figsize=(15, 5 * D), sharex=True)
    fig.suptitle("Action Comparison for lerobot", fontsize=16)
    for i in range(D):
        ax = axs[i] if D > 1 else axs
        ax.plot(range(gt.shape[0]), gt[:, i].numpy(), label="Ground Truth")
        ax.plot(range(gt.shape[0]), pred[:, i].numpy(), label="Prediction")
        ax.set_ylabel(f"Action Dim {i + 1}")
        ax.legend()
        ax.grid(True)
    out = os.path.join(save_dir, "lerobot_comparison.png")
    plt.tight_layout(rect=[0, 0.03, 1, 0.95])
    plt.savefig(out)
    plt.close()
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="")
    ap.add_argument("--action-tokenizer", default=None)
    ap.add_argument("--config", default="", help="training YAML (data section is used)")
    ap.add_argument("--save-dir", required=True)
    ap.add_argument("--pred-horizon", type=int, default=32)
    ap.add_argument("--action-dim", type=int, default=14)
    ap.add_argument("--predict-mode", default="fast", choices=["fast", "diffusion"])
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--frames", type=int, default=40, help="synthetic: episode length")
    ap.add_argument("--device", default="auto")
    args = ap.parse_args(argv)
    dev = pick_device(args.device)
    model = load_model(args.model, args.synthetic, dev, args.action_tokenizer, use_fast_tokenizer=(args.predict_mode == "fast"))
    from ..data.lerobot import SyntheticEpisodeDataset, get_data_configs, load_test_dataset

    if args.synthetic:
        config = {"batch_size_per_gpu": 1, "num_workers": 0, "use_fast_tokenizer": args.predict_mode == "fast",
                  "data": {"action_horizon": args.pred_horizon,
                           "resolution": {"face_view": 112, "left_wrist_view": 112, "right_wrist_view": 112}}}
        ds = SyntheticEpisodeDataset(n=args.frames, horizon=args.pred_horizon, action_dim=args.action_dim)
        dataset = load_test_dataset(config, {}, dataset=ds, processor=model.processor, model_config=model.config)
    else:
        import yaml

        with open(args.config) as f:
            config = yaml.safe_load(f)
        config["data"]["model_type"] = config.get("model_type")
        lerobot_config = get_data_configs(config["data"]).get("lerobot_config", {})
        dataset = load_test_dataset(config, lerobot_config, seed=42, processor=model.processor,
                                    action_tokenizer=getattr(model, "action_tokenizer", None), model_config=model.config)
    gt, pred = rollout(model, dataset.get_dataloader(), args.pred_horizon, args.action_dim, args.predict_mode)
    out = plot(args.save_dir, gt, pred)
    print("wrote", out)
    return 0


if __name__ == "__main__":
    sys.exit(main())

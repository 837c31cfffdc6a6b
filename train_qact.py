"""Training entry point: ``python train_qact.py --config config.yml --seed 42``.

Single GPU: run it directly. Several GPUs of one node: ``torchrun --standalone --local-addr
127.0.0.1 --nproc-per-node N train_qact.py --config ...`` (one process per GPU). Accepts the
reference's YAML (workspace/lerobot_example/config_qact.yml); see ``wallx_b200/train/trainer.py``
for the few extra keys. Reference entry point: train_qact.py:106-142.
"""
import argparse
import os
import sys

import yaml

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def load_config(path: str) -> dict:
    with open(path, "r", encoding="utf-8") as f:
        config = yaml.safe_load(f)
    config.setdefault("data", {})
    config["data"]["model_type"] = config.get("model_type", "qwen2_5")
    return config


def setup_distributed():
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1 and not torch.distributed.is_initialized():
        backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {"device_id": torch.device("cuda", torch.cuda.current_device())} if backend == "nccl" else {}
        torch.distributed.init_process_group(backend, **kw)
    return world


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=str, required=True)
    ap.add_argument("--seed", type=int, default=42)
    args = ap.parse_args(argv)
    config = load_config(args.config)
    setup_distributed()
    from wallx_b200.train.trainer import QwenVlAct_Trainer

    if int(os.environ.get("RANK", "0")) == 0:
        if config.get("save_path"):
            os.makedirs(config["save_path"], exist_ok=True)
        print("configuration:")
        for k, v in config.items():
            print(f"  {k}: {v}")
    trainer = QwenVlAct_Trainer(config=config, logger=None, accelerator=None, seed=args.seed)
    trainer.fit()
    import torch

    if torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()

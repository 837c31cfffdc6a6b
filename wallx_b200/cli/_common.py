"""Shared model/processor loading for the command-line tools."""
from __future__ import annotations

import torch


def pick_device(name: str = "auto") -> torch.device:
    if name == "auto":
        return torch.device("cuda" if torch.cuda.is_available() else "cpu")
    return torch.device(name)


def load_model(model_path: str | None, synthetic: bool, device: torch.device, action_tokenizer_path=None,
               use_fast_tokenizer: bool = False):
    """``from_pretrained`` on a checkpoint directory, or a tiny random model when ``synthetic``."""
    from ..models import Qwen2_5_VLMoEForAction

    if synthetic or not model_path:
        from ..config import tiny_config
        from ..data.synthetic import make_processor

        # 20-d action / proprioception like the released model (the collator pads both to 20)
        cfg = tiny_config(dof_config={"arm": 20}, agent_pos_config={"arm": 20})
        proc = make_processor(cfg, 16)
        torch.manual_seed(0)
        model = Qwen2_5_VLMoEForAction(cfg, processor=proc, use_fast_tokenizer=use_fast_tokenizer)
        model.init_weights(seed=0)
    else:
        model = Qwen2_5_VLMoEForAction.from_pretrained(model_path, action_tokenizer_path=action_tokenizer_path)
    model.eval()
    if device.type == "cuda":
        model = model.to(device).to(torch.bfloat16)
    return model

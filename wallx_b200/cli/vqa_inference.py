"""Visual question answering with greedy decoding (reference: scripts/vqa_inference.py:8-84).

``python -m wallx_b200.cli.vqa_inference --model DIR --image frame.png --question "..."``; with
``--synthetic`` a tiny random model answers from the synthetic processor's vocabulary.
"""
from __future__ import annotations

import argparse
import sys

import torch

from ._common import load_model, pick_device


class VQAWrapper:
    def __init__(self, model_path: str = "", synthetic: bool = False, device: str = "auto"):
        self.device = pick_device(device)
        self.model = load_model(model_path, synthetic, self.device)
        self.processor = self.model.processor

    def generate(self, image, text: str, **kwargs) -> str:
        messages = [{"role": "user", "content": [{"type": "image"}, {"type": "text", "text": text}]}]
        prompt = self.processor.apply_chat_template(messages, tokenize=False, add_generation_prompt=True)
        inputs = self.processor(text=[prompt], images=[image], return_tensors="pt")
        float_dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        inputs = {k: (v.to(self.device, float_dtype) if torch.is_tensor(v) and v.is_floating_point()
                      else (v.to(self.device) if torch.is_tensor(v) else v)) for k, v in inputs.items()}
        tok = self.processor.tokenizer
        params = {"max_new_tokens": 1024, "do_sample": False, "eos_token_id": tok.eos_token_id,
                  "pad_token_id": tok.pad_token_id, **kwargs}
        with torch.no_grad():
            out = self.model.generate(**inputs, **params)
        new = [o[len(i):] for i, o in zip(inputs["input_ids"], out)]
        return self.processor.batch_decode(new, skip_special_tokens=True, clean_up_tokenization_spaces=False)[0]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--image", default="")
    ap.add_argument("--question", default="What should the robot do next? Think step by step.")
    ap.add_argument("--max-new-tokens", type=int, default=1024)
    ap.add_argument("--device", default="auto")
    args = ap.parse_args(argv)
    w = VQAWrapper(args.model, args.synthetic, args.device)
    if args.image:
        from PIL import Image

        img = Image.open(args.image).convert("RGB")
    else:
        img = torch.randint(0, 256, (112, 112, 3), dtype=torch.uint8)
    print("model answer:", w.generate(img, args.question, max_new_tokens=args.max_new_tokens))
    return 0


if __name__ == "__main__":
    sys.exit(main())

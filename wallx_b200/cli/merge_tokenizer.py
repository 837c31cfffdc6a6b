"""Add the action vocabulary to a Qwen2.5-VL processor and save it
(reference: scripts/merge_tokenizer.py:1-26).

Adds ``<|propri|>``, ``<|action|>`` and ``<|action_token_i|>`` for every id of the FAST action
tokenizer, records ``action_token_start_index`` / ``action_token_vocab_size`` in the tokenizer's
``init_kwargs`` and writes the processor to ``--out``. ``--synthetic N`` does the same on the
in-repo synthetic processor with an N-id action vocabulary (no files needed).
"""
from __future__ import annotations

import argparse
import sys


def merge(processor, action_vocab_size: int):
    new_tokens = ["<|propri|>", "<|action|>"] + [f"<|action_token_{i}|>" for i in range(action_vocab_size)]
    added = processor.tokenizer.add_tokens(new_tokens)
    start = processor.tokenizer.convert_tokens_to_ids("<|action_token_0|>")
    processor.tokenizer.init_kwargs["action_token_start_index"] = start
    processor.tokenizer.init_kwargs["action_token_vocab_size"] = action_vocab_size
    return added, start


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--processor", default="", help="directory of the Qwen2.5-VL processor")
    ap.add_argument("--action-tokenizer", default="", help="directory of the FAST action tokenizer")
    ap.add_argument("--out", required=True)
    ap.add_argument("--synthetic", type=int, default=0, help="use the synthetic processor with this many action ids")
    args = ap.parse_args(argv)
    if args.synthetic:
        from ..data.synthetic import SyntheticProcessor, SyntheticTokenizer

        tok = SyntheticTokenizer(1000, 0, 990, 991, 992, 993)
        del tok.special["<|propri|>"], tok.special["<|action|>"]
        tok._len = tok.action_start = 1000
        processor, n_act = SyntheticProcessor(tok), args.synthetic
    else:
        from transformers import AutoProcessor

        processor = AutoProcessor.from_pretrained(args.processor, use_fast=True)
        processor.tokenizer.padding_side = "left"
        n_act = AutoProcessor.from_pretrained(args.action_tokenizer, trust_remote_code=True).vocab_size
    added, start = merge(processor, n_act)
    processor.save_pretrained(args.out)
    print(f"added {added} tokens; action_token_start_index={start}; action_token_vocab_size={n_act}; saved to {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())

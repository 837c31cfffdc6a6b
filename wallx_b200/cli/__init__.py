"""Command-line tools (``python -m wallx_b200.cli.<name>``): fake_inference, vqa_inference,
draw_openloop_plot, merge_tokenizer. Each mirrors one of the reference's ``scripts/*.py`` and
adds a ``--synthetic`` mode that needs no checkpoint (tiny random model + synthetic processor)."""

from wallx_b200.train.trainer import QwenVlAct_Trainer, print_rank_last, seed_all, timer  # noqa: F401

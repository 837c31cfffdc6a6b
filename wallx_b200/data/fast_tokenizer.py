"""A self-contained FAST-style action tokenizer (DCT along time, uniform quantisation, zero-run
truncation) with the call surface of the Hugging Face ``physical-intelligence/fast`` processor that
the reference loads with ``AutoProcessor.from_pretrained(action_tokenizer_path,
trust_remote_code=True)`` (wall_x/data/load_lerobot_dataset.py:283-286, wall_x/data/utils.py:506-530,
modeling_qwen2_5_vl_act.py:1840-1884):

* ``tok(actions)`` with ``actions [B, T, D]`` (or ``[T, D]``) in ``[-1, 1]`` -> ``List[List[int]]``
* ``tok.decode(list_of_id_lists, time_horizon=T, action_dim=D)`` -> ``np.ndarray [B, T, D]`` (an
  all-zero chunk when the ids cannot be decoded, which callers treat as "no prediction")
* ``tok.vocab_size``

The pretrained FAST tokenizer additionally BPE-compresses the coefficient stream; checkpoints trained
with it must keep using it (pass its directory as ``action_tokenizer_path``). This one needs no
files, so FAST-mode training, inference and the tools run end to end without downloads.
"""
from __future__ import annotations

import math
from typing import List, Sequence

import numpy as np


def _dct_matrix(n: int) -> np.ndarray:
    """Orthonormal DCT-II matrix ``C`` with ``coeff = C @ x``; ``C.T`` inverts it."""
    k = np.arange(n)[:, None]
    t = np.arange(n)[None, :]
    c = np.cos(math.pi * (2 * t + 1) * k / (2 * n)) * math.sqrt(2.0 / n)
    c[0] *= 1.0 / math.sqrt(2.0)
    return c


class DctActionTokenizer:
    def __init__(self, vocab_size: int = 2048, scale: float = 10.0):
        if vocab_size < 3:
            raise ValueError("vocab_size must be at least 3")
        self.vocab_size = int(vocab_size)
        self.scale = float(scale)
        self.zero = self.vocab_size // 2  # id of a zero coefficient
        self._cache = {}

    def _mat(self, n: int) -> np.ndarray:
        if n not in self._cache:
            self._cache[n] = _dct_matrix(n)
        return self._cache[n]

    def __call__(self, actions) -> List[List[int]]:
        a = np.asarray(actions, dtype=np.float64)
        if a.ndim == 2:
            a = a[None]
        out = []
        for chunk in a:
            coeff = self._mat(chunk.shape[0]) @ chunk  # [T, D], row k = frequency k of every dimension
            q = np.rint(coeff * self.scale).astype(np.int64) + self.zero
            q = np.clip(q, 0, self.vocab_size - 1).reshape(-1)  # low frequencies first
            nz = np.nonzero(q != self.zero)[0]
            end = int(nz[-1]) + 1 if nz.size else 1
            out.append(q[:end].tolist())
        return out

    def decode(self, tokens: Sequence[Sequence[int]], time_horizon: int, action_dim: int) -> np.ndarray:
        res = np.zeros((len(tokens), time_horizon, action_dim), dtype=np.float32)
        n = time_horizon * action_dim
        for b, ids in enumerate(tokens):
            ids = [int(i) for i in ids]
            if not ids or len(ids) > n or any(i < 0 or i >= self.vocab_size for i in ids):
                continue
            q = np.full(n, self.zero, dtype=np.float64)
            q[: len(ids)] = ids
            coeff = (q - self.zero).reshape(time_horizon, action_dim) / self.scale
            res[b] = (self._mat(time_horizon).T @ coeff).astype(np.float32)
        return res

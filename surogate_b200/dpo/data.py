"""Preference rows -> padded (prompt + answer) token rows with targets masked on the prompt.

Each pair becomes two rows of ``sequence_len`` tokens (chosen first, rejected second); targets are the inputs shifted by
one, -100 on the prompt and on padding, so that sum(log p(target)) over a row is log p(answer | prompt).

Parity: surogate/dpo/data.py.
"""
from __future__ import annotations

from typing import Any, Dict, List, Sequence, Tuple

import numpy as np

IGNORE = -100


def encode_pair(tok, row: Dict[str, Any], seq_len: int, max_prompt_len: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray, np.ndarray]:
    prompt_text = tok.apply_chat_template(row["prompt"], add_generation_prompt=True, enable_thinking=row.get("enable_thinking"))
    p = tok.encode(prompt_text)[-max_prompt_len:]
    eos = [tok.eos_token_id] if tok.eos_token_id >= 0 else []

    def one(answer: str):
        a = tok.encode(answer) + eos
        ids = (p + a)[: seq_len + 1]
        x = np.full(seq_len + 1, tok.pad_token_id if tok.pad_token_id >= 0 else 0, np.int32)
        x[:len(ids)] = ids
        y = np.full(seq_len, IGNORE, np.int32)
        lo, hi = max(len(p) - 1, 0), len(ids) - 1
        y[lo:hi] = x[lo + 1:hi + 1]
        return x[:-1], y

    xc, yc = one(row["chosen"])
    xr, yr = one(row["rejected"])
    return xc, yc, xr, yr


def build_pairs(tok, rows: Sequence[Dict[str, Any]], seq_len: int, max_prompt_len: int):
    X, Y = [], []
    for r in rows:
        xc, yc, xr, yr = encode_pair(tok, r, seq_len, max_prompt_len)
        if (yc != IGNORE).any() and (yr != IGNORE).any():
            X += [xc, xr]
            Y += [yc, yr]
    return np.stack(X) if X else np.zeros((0, seq_len), np.int32), np.stack(Y) if Y else np.zeros((0, seq_len), np.int32)


class PairLoader:
    """Serves ``pairs_per_step`` pairs (2 rows each: chosen, rejected) per call, shuffled per epoch, strided over ranks."""

    def __init__(self, X: np.ndarray, Y: np.ndarray, pairs_per_step: int, seed: int = 0, rank: int = 0, world: int = 1):
        assert X.shape[0] % 2 == 0
        self.X, self.Y, self.n, self.k = X, Y, X.shape[0] // 2, pairs_per_step
        self.seed, self.rank, self.world = seed, rank, world
        self.epoch, self.cursor = 0, 0
        self._order = self._make_order()
        if len(self._order) < self.k:
            raise ValueError(f"only {len(self._order)} preference pairs for this rank, fewer than one step ({self.k})")

    def _make_order(self):
        return np.random.default_rng([self.seed, self.epoch]).permutation(self.n)[self.rank::self.world]

    def steps_per_epoch(self) -> int:
        return len(self._order) // self.k

    def next(self):
        if self.cursor + self.k > len(self._order):
            self.epoch += 1
            self.cursor = 0
            self._order = self._make_order()
        idx = self._order[self.cursor:self.cursor + self.k]
        self.cursor += self.k
        rows = np.stack([2 * idx, 2 * idx + 1], axis=1).reshape(-1)
        return self.X[rows], self.Y[rows]

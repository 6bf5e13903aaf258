"""Where does the training signal of a multi-turn rollout live along its turns?

``TurnStats`` collects, per turn index, over the supervised tokens of a step: the signed and the absolute per-token KL estimate
(new vs behaviour log-prob), the realised loss, the token count and how many samples reached that turn.  From those it reports
per-turn means and each turn's share of tokens, of |KL| and of loss, plus deep-versus-shallow ratios (last third of the turns
against the first third).  Shares use magnitudes: the signed KL estimate changes sign along the turns, so its sum is no budget.
``turn_weights`` gives the per-token weights that move a trajectory-level token average (alpha = 0) towards equal weight per
turn (alpha = 1) while keeping the total weight, for reporting the counterfactual or for use as ``row_weights``.

Turn ids come from the packer's completion mask: tokens the policy produced between two environment segments share a turn.

Parity: surogate/grpo/turn_stats.py (TurnAccumulator, blend_weight).
"""
from __future__ import annotations

from collections import defaultdict
from typing import Dict, List, Optional

import numpy as np


def turn_ids_from_mask(completion_mask: np.ndarray) -> np.ndarray:
    """1 = policy token, 0 = environment token -> turn index per token (-1 on environment tokens); a new turn starts at every
    0 -> 1 edge."""
    m = np.asarray(completion_mask).astype(bool)
    starts = m & ~np.concatenate([[False], m[:-1]])
    ids = np.cumsum(starts) - 1
    return np.where(m, ids, -1).astype(np.int32)


class TurnStats:
    def __init__(self):
        self.kl = defaultdict(float)
        self.abs_kl = defaultdict(float)
        self.loss = defaultdict(float)
        self.tokens = defaultdict(int)
        self.reached = defaultdict(int)
        self.samples = 0

    def add_sample(self, turn_ids: np.ndarray, mask: np.ndarray, logp_new: np.ndarray, logp_old: np.ndarray, token_loss: Optional[np.ndarray] = None) -> None:
        """One sample's token arrays (same length).  ``mask``: supervised tokens."""
        turn_ids, mask = np.asarray(turn_ids), np.asarray(mask).astype(bool) & (np.asarray(turn_ids) >= 0)
        if not mask.any():
            return
        self.samples += 1
        d = (np.asarray(logp_new, np.float64) - np.asarray(logp_old, np.float64))[mask]
        t = turn_ids[mask]
        l = np.asarray(token_loss, np.float64)[mask] if token_loss is not None else np.zeros_like(d)
        for turn in np.unique(t):
            sel = t == turn
            k = int(turn)
            self.kl[k] += float(d[sel].sum())
            self.abs_kl[k] += float(np.abs(d[sel]).sum())
            self.loss[k] += float(np.abs(l[sel]).sum())
            self.tokens[k] += int(sel.sum())
            self.reached[k] += 1

    def turns(self) -> List[int]:
        return sorted(self.tokens)

    def _share(self, table) -> Dict[int, float]:
        total = sum(table[t] for t in self.turns())
        return {t: (table[t] / total if total > 0 else 0.0) for t in self.turns()}

    def rows(self) -> List[Dict[str, float]]:
        tok, kls, ls = self._share(self.tokens), self._share(self.abs_kl), self._share(self.loss)
        return [{"turn": t, "tokens": self.tokens[t], "survivors": self.reached[t], "mean_kl": self.kl[t] / self.tokens[t],
                 "mean_abs_kl": self.abs_kl[t] / self.tokens[t], "token_share": tok[t], "abs_kl_share": kls[t], "loss_share": ls[t]} for t in self.turns()]

    def summary(self) -> Dict[str, float]:
        ts = self.turns()
        out = {"turns/max_depth": float(len(ts)), "turns/samples": float(self.samples)}
        if len(ts) < 3:
            return out
        third = max(1, len(ts) // 3)
        shallow, deep = ts[:third], ts[-third:]

        def mean(table, which):
            n = sum(self.tokens[t] for t in which)
            return sum(table[t] for t in which) / n if n else 0.0

        out["turns/deep_over_shallow_abs_kl"] = mean(self.abs_kl, deep) / max(mean(self.abs_kl, shallow), 1e-12)
        out["turns/deep_token_share"] = sum(self._share(self.tokens)[t] for t in deep)
        out["turns/deep_abs_kl_share"] = sum(self._share(self.abs_kl)[t] for t in deep)
        out["turns/deep_loss_share"] = sum(self._share(self.loss)[t] for t in deep)
        out["turns/deep_survivor_fraction"] = min(self.reached[t] for t in deep) / max(1, self.samples)
        return out


def turn_weights(turn_ids: np.ndarray, mask: np.ndarray, alpha: float) -> np.ndarray:
    """Per-token weights: (1 - alpha) x (every token equal) + alpha x (every turn equal), scaled so they sum to the number of
    supervised tokens."""
    turn_ids = np.asarray(turn_ids)
    sup = np.asarray(mask).astype(bool) & (turn_ids >= 0)
    w = np.zeros(turn_ids.shape, np.float32)
    n = int(sup.sum())
    if n == 0:
        return w
    uniq, counts = np.unique(turn_ids[sup], return_counts=True)
    T = len(uniq)
    for t, c in zip(uniq, counts):
        w[sup & (turn_ids == t)] = (1.0 - alpha) / n + alpha / (T * c)
    return w * (n / w.sum())

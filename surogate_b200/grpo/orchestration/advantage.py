"""Advantage functions: rewards of one prompt's group of rollouts -> one advantage per rollout.

``default``  reward minus the group mean (optionally the completion-length-weighted mean, which removes the bias towards long
             completions when the loss is token-normalised);
``std``      the same divided by the group's standard deviation (classic GRPO).
Groups whose rewards are all equal get zero advantages (no signal); the caller may drop them.

Parity: surogate/grpo/orchestrator/advantage.py:36-104.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np


@dataclass
class AdvantageInputs:
    rewards: np.ndarray            # [prompts, group]
    completion_lengths: np.ndarray  # [prompts, group]


@dataclass
class AdvantageOutputs:
    advantages: np.ndarray         # [prompts, group]


def default_advantage(inp: AdvantageInputs, length_weighted_mean: bool = False) -> AdvantageOutputs:
    r = inp.rewards.astype(np.float64)
    if length_weighted_mean:
        w = np.maximum(inp.completion_lengths.astype(np.float64), 1.0)
        base = (r * w).sum(1, keepdims=True) / w.sum(1, keepdims=True)
    else:
        base = r.mean(1, keepdims=True)
    return AdvantageOutputs((r - base).astype(np.float32))


def std_normalized_advantage(inp: AdvantageInputs, eps: float = 1e-4) -> AdvantageOutputs:
    r = inp.rewards.astype(np.float64)
    return AdvantageOutputs(((r - r.mean(1, keepdims=True)) / (r.std(1, keepdims=True) + eps)).astype(np.float32))


ADVANTAGE_FNS: Dict[str, Callable[..., AdvantageOutputs]] = {"default": default_advantage, "std": std_normalized_advantage}


def compute_advantages(rewards: Sequence[float], completion_lengths: Sequence[int], group_size: int, kind: str = "default",
                       custom: Optional[Callable[[AdvantageInputs], AdvantageOutputs]] = None, **kw) -> List[float]:
    """Flat lists (prompt-major, ``group_size`` rollouts per prompt) in, flat list of advantages out.  ``custom`` (or a
    ``module:function`` string as ``kind``) plugs in a user function with the same input / output records."""
    r = np.asarray(rewards, dtype=np.float32).reshape(-1, group_size)
    n = np.asarray(completion_lengths, dtype=np.int64).reshape(-1, group_size)
    fn = custom
    if fn is None:
        if ":" in kind:
            import importlib

            mod, name = kind.split(":", 1)
            fn = getattr(importlib.import_module(mod), name)
        else:
            fn = ADVANTAGE_FNS[kind]
    out = fn(AdvantageInputs(r, n), **kw)
    return [float(x) for x in np.asarray(out.advantages).reshape(-1)]

"""Periodic evaluation of the current policy on held-out examples of the training environment.

Every ``eval_every`` steps the orchestrator samples ``n`` completions per held-out example through the same ``generate_group``
callable that produces training rollouts (so single- and multi-turn environments are evaluated the way they are trained) and
reports the mean reward, pass@1 and pass@k (unbiased estimator: 1 - C(n - c, k) / C(n, k) with c = completions whose reward
reaches ``pass_threshold``), the mean completion length and the share of examples no completion solves.  Evaluation rollouts never
enter the buffer or the trainer batch.

Parity: surogate/grpo/orchestrator/eval_utils.py.
"""
from __future__ import annotations

from math import comb
from typing import Any, Callable, Dict, List, Sequence


def pass_at_k(n: int, c: int, k: int) -> float:
    if n <= 0 or k <= 0:
        return 0.0
    k = min(k, n)
    if n - c < k:
        return 1.0
    return 1.0 - comb(n - c, k) / comb(n, k)


def evaluate_policy(examples: Sequence[Dict[str, Any]], generate_group: Callable[..., List[Any]], n_samples: int, sampling: Dict[str, Any], policy_version: int = 0,
                    ks: Sequence[int] = (1, 8), pass_threshold: float = 1.0, num_servers: int = 1) -> Dict[str, float]:
    rewards: List[float] = []
    lengths: List[int] = []
    per_example = []
    for i, ex in enumerate(examples):
        group = generate_group(ex, n_samples, dict(sampling), policy_version, i % max(1, num_servers))
        rs = [float(r.reward) for r in group]
        rewards += rs
        lengths += [len(r.completion_ids) for r in group]
        per_example.append((len(rs), sum(r >= pass_threshold for r in rs)))
    out = {"eval/examples": float(len(examples)), "eval/mean_reward": sum(rewards) / max(1, len(rewards)),
           "eval/completion_len": sum(lengths) / max(1, len(lengths)),
           "eval/unsolved_fraction": sum(1 for n, c in per_example if c == 0) / max(1, len(per_example))}
    for k in ks:
        vals = [pass_at_k(n, c, k) for n, c in per_example if n > 0]
        out[f"eval/pass@{k}"] = sum(vals) / max(1, len(vals))
    return out

"""Rollout filters: degenerate completions are detected from the sampled token ids and their behaviour log-probs and are masked
out of the loss (their reward is kept for the group statistics).

``GibberishFilter``   flags a rollout whose mean per-token surprise is close to that of uniform sampling over the vocabulary
                      (the policy was sampling noise: entropy collapse the other way round); with ``token_id_threshold`` it uses
                      the per-token rule instead: one rare token (id above the threshold) sampled at a log-prob below
                      ``-log(vocab) - logprob_offset`` flags the rollout;
``RepetitionFilter``  flags a rollout that repeats the same n-gram many times in a row or spends most of its tokens on a few
                      distinct n-grams; with ``window`` / ``prob_threshold`` it uses the confidence-streak rule instead: ``window``
                      consecutive tokens each sampled with probability above ``prob_threshold``.

``enforce`` (default true) decides whether a detection clears the completion mask or is only counted.

Parity: surogate/grpo/orchestrator/filters.py:36-183.
"""
from __future__ import annotations

import math
from collections import Counter
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Protocol, Sequence


@dataclass
class FilterResult:
    detected: bool
    detail: str = ""


class RolloutFilter(Protocol):
    name: str

    def check(self, rollout) -> FilterResult: ...


class GibberishFilter:
    name = "gibberish"

    def __init__(self, vocab_size: int, logprob_offset: float = 2.0, min_tokens: int = 16, token_id_threshold: Optional[int] = None,
                 enforce: bool = True):
        """A completion is gibberish when its mean token log-prob is below ``-(log(vocab) - logprob_offset)``; with
        ``token_id_threshold``, when one token with a larger id was sampled below ``-log(vocab) - logprob_offset``."""
        self.token_id_threshold, self.enforce = token_id_threshold, enforce
        self.threshold = -(math.log(max(2, vocab_size)) - logprob_offset)
        self.token_threshold = -math.log(max(2, vocab_size)) - logprob_offset
        self.min_tokens = min_tokens

    def check(self, rollout) -> FilterResult:
        if self.token_id_threshold is not None:
            for i, (t, l) in enumerate(zip(rollout.completion_ids, rollout.logprobs)):
                if t > self.token_id_threshold and l < self.token_threshold:
                    return FilterResult(True, f"rare token {t} at position {i} sampled at logprob {l:.2f}")
            return FilterResult(False)
        lp = list(rollout.logprobs)
        if len(lp) < self.min_tokens:
            return FilterResult(False)
        mean = sum(lp) / len(lp)
        return FilterResult(mean < self.threshold, f"mean logprob {mean:.2f} < {self.threshold:.2f}")


class RepetitionFilter:
    name = "repetition"

    def __init__(self, ngram: int = 8, max_consecutive: int = 6, max_top_fraction: float = 0.5, min_tokens: int = 64, window: Optional[int] = None,
                 prob_threshold: float = 0.99, enforce: bool = True):
        self.n, self.max_consecutive, self.max_top_fraction, self.min_tokens = ngram, max_consecutive, max_top_fraction, min_tokens
        self.window, self.streak_logprob, self.enforce = window, math.log(prob_threshold), enforce

    def check(self, rollout) -> FilterResult:
        if self.window is not None:
            streak = 0
            for i, l in enumerate(rollout.logprobs):
                streak = streak + 1 if l > self.streak_logprob else 0
                if streak >= self.window:
                    return FilterResult(True, f"{streak} consecutive tokens above the confidence threshold, ending at position {i}")
            return FilterResult(False)
        ids = list(rollout.completion_ids)
        if len(ids) < max(self.min_tokens, 2 * self.n):
            return FilterResult(False)
        grams = [tuple(ids[i:i + self.n]) for i in range(0, len(ids) - self.n + 1)]
        # the same n-gram at stride n, many times in a row
        run = best = 1
        for i in range(self.n, len(grams), self.n):
            run = run + 1 if grams[i] == grams[i - self.n] else 1
            best = max(best, run)
        if best >= self.max_consecutive:
            return FilterResult(True, f"{best} consecutive repeats of one {self.n}-gram")
        top = Counter(grams).most_common(1)[0][1] * self.n / len(ids)
        return FilterResult(top > self.max_top_fraction, f"one {self.n}-gram covers {top:.0%} of the completion")


def make_filters(configs: Sequence[Dict[str, Any]], vocab_size: int) -> List[RolloutFilter]:
    out: List[RolloutFilter] = []
    for c in configs or []:
        c = dict(c)
        kind = c.pop("type")
        if kind == "gibberish":
            out.append(GibberishFilter(vocab_size, **c))
        elif kind == "repetition":
            out.append(RepetitionFilter(**c))
        else:
            raise ValueError(f"unknown rollout filter '{kind}' (gibberish | repetition)")
    return out


def apply_filters(filters: Sequence[RolloutFilter], rollouts: Sequence) -> Dict[str, float]:
    """Marks flagged rollouts (``meta['filtered'] = name``; the completion mask is zeroed, so they add nothing to the loss, unless
    the filter says ``enforce=False``) and returns per-filter detection rates.  The first matching filter wins."""
    stats = {f"filter/{f.name}": 0.0 for f in filters}
    for r in rollouts:
        for f in filters:
            res = f.check(r)
            if res.detected:
                r.meta["filtered"] = f.name
                r.meta["filter_detail"] = res.detail
                if getattr(f, "enforce", True):
                    r.completion_mask = [0] * len(r.completion_ids)
                stats[f"filter/{f.name}"] += 1.0
                break
    n = max(1, len(rollouts))
    return {k: v / n for k, v in stats.items()}

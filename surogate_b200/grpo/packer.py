"""Pack variable-length rollouts into fixed [rows, T] micro-batches for the trainer.

A rollout = prompt ids + completion ids + per-completion-token behaviour log-probs + one advantage.  Samples are placed
first-fit-decreasing into rows of T tokens; within a row position ids restart per sample (so attention is block-diagonal
causal), targets are inputs shifted by one inside a sample, and the loss mask / advantages / old log-probs are aligned to
the *target* position (the token being predicted).  Unused space is padding with target -100.

Parity: surogate/grpo/packer.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Dict, List, Sequence

import numpy as np

IGNORE = -100


@dataclass
class Rollout:
    prompt_ids: List[int]
    completion_ids: List[int]
    logprobs: List[float]        # behaviour policy log-prob of each completion token
    advantage: float = 0.0
    reward: float = 0.0
    policy_version: int = 0
    group: int = 0
    meta: Dict = field(default_factory=dict)
    # multi-turn rollouts: 1 for tokens the policy produced, 0 for environment tokens (tool results, turn markers) that sit
    # between its turns; None means every completion token is the policy's
    completion_mask: Optional[List[int]] = None
    # log-prob of each completion token under a teacher model (``loss.teacher_tau``); None when no teacher scored the rollout
    teacher_logprobs: Optional[List[float]] = None

    def __len__(self) -> int:
        return len(self.prompt_ids) + len(self.completion_ids)


@dataclass
class PackedBatch:
    inputs: np.ndarray        # int32 [rows, T]
    targets: np.ndarray       # int32 [rows, T]   (-100 = no loss)
    position_ids: np.ndarray  # int32 [rows, T]
    advantages: np.ndarray    # float32 [rows, T]
    old_logprobs: np.ndarray  # float32 [rows, T]
    seq_ids: np.ndarray       # int32 [rows, T]   (-1 = padding)
    policy_version: int = 0
    n_samples: int = 0
    teacher_logprobs: Optional[np.ndarray] = None   # float32 [rows, T], present when every packed rollout carries teacher scores

    def arrays(self) -> Dict[str, np.ndarray]:
        out = {"inputs": self.inputs, "targets": self.targets, "position_ids": self.position_ids, "advantages": self.advantages,
               "old_logprobs": self.old_logprobs, "seq_ids": self.seq_ids}
        if self.teacher_logprobs is not None:
            out["teacher_logprobs"] = self.teacher_logprobs
        return out


def _truncate(r: Rollout, T: int) -> Rollout:
    if len(r) <= T:
        return r
    keep_c = max(1, T - len(r.prompt_ids))
    if keep_c < len(r.completion_ids) and len(r.prompt_ids) < T:
        return Rollout(r.prompt_ids, r.completion_ids[:keep_c], r.logprobs[:keep_c], r.advantage, r.reward, r.policy_version, r.group, r.meta,
                       r.completion_mask[:keep_c] if r.completion_mask is not None else None,
                       r.teacher_logprobs[:keep_c] if r.teacher_logprobs is not None else None)
    p = r.prompt_ids[-(T - 1):]
    return Rollout(p, r.completion_ids[:1], r.logprobs[:1], r.advantage, r.reward, r.policy_version, r.group, r.meta,
                   r.completion_mask[:1] if r.completion_mask is not None else None, r.teacher_logprobs[:1] if r.teacher_logprobs is not None else None)


def pack_rollouts(rollouts: Sequence[Rollout], seq_len: int, rows: int, pad_id: int = 0) -> List[PackedBatch]:
    """Pack into as many batches of ``rows`` rows as needed (the last one is padded with empty rows).  ``rows <= 0``: one batch
    with exactly as many rows as the samples need (the trainer pads it to a multiple of its micro-batch)."""
    T = seq_len
    samples = [_truncate(r, T) for r in rollouts if r.completion_ids]
    order = sorted(range(len(samples)), key=lambda i: -len(samples[i]))
    bins: List[List[int]] = []
    space: List[int] = []
    for i in order:
        n = len(samples[i])
        for b, free in enumerate(space):
            if free >= n:
                bins[b].append(i)
                space[b] -= n
                break
        else:
            bins.append([i])
            space.append(T - n)
    if rows <= 0:
        rows = max(1, len(bins))
    while len(bins) % rows != 0 or not bins:
        bins.append([])
    out: List[PackedBatch] = []
    sid = 0
    with_teacher = bool(samples) and all(s.teacher_logprobs is not None and len(s.teacher_logprobs) == len(s.completion_ids) for s in samples)
    for b0 in range(0, len(bins), rows):
        R = rows
        x = np.full((R, T), pad_id, np.int32)
        y = np.full((R, T), IGNORE, np.int32)
        pos = np.zeros((R, T), np.int32)
        adv = np.zeros((R, T), np.float32)
        old = np.zeros((R, T), np.float32)
        seq = np.full((R, T), -1, np.int32)
        teach = np.zeros((R, T), np.float32) if with_teacher else None
        n_samples, version = 0, None
        for r, members in enumerate(bins[b0:b0 + rows]):
            at = 0
            for i in members:
                s = samples[i]
                ids = np.asarray(s.prompt_ids + s.completion_ids, np.int32)
                n, P = len(ids), len(s.prompt_ids)
                x[r, at:at + n] = ids
                pos[r, at:at + n] = np.arange(n)
                # position j predicts token j+1: completion token c (index P+c) is the target at position P+c-1
                lo, hi = at + P - 1, at + n - 1
                if P == 0:  # no prompt: the first completion token has no context to be predicted from
                    lo += 1
                    y[r, lo:hi] = ids[1:]
                    old[r, lo:hi] = np.asarray(s.logprobs[1:], np.float32)
                    if teach is not None:
                        teach[r, lo:hi] = np.asarray(s.teacher_logprobs[1:], np.float32)
                else:
                    y[r, lo:hi] = ids[P:]
                    old[r, lo:hi] = np.asarray(s.logprobs, np.float32)
                    if teach is not None:
                        teach[r, lo:hi] = np.asarray(s.teacher_logprobs, np.float32)
                adv[r, lo:hi] = s.advantage
                if s.completion_mask is not None:  # environment tokens are context only
                    m = np.asarray(s.completion_mask[(1 if P == 0 else 0):], bool)
                    y[r, lo:hi][~m] = IGNORE
                    adv[r, lo:hi][~m] = 0.0
                seq[r, at:at + n] = sid
                sid += 1
                at += n
                n_samples += 1
                version = s.policy_version if version is None else min(version, s.policy_version)
            pos[r, at:] = np.arange(T - at)
        out.append(PackedBatch(x, y, pos, adv, old, seq, version or 0, n_samples, teach))
    return out

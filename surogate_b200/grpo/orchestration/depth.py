"""Adaptive rollout-depth budgeting for multi-turn environments.

Most of a multi-turn rollout's wall clock is spent on a few very deep episodes that seldom earn reward.  The controller observes
(depth, reward) of finished rollouts and sets a depth cap at a quantile of the depths that were actually needed by rewarded
rollouts (times a head-room factor); every ``probe_every``-th step runs uncapped so that the estimate can grow again when the
policy starts needing more turns.  The reference reports 1.36x wall clock from this (RELEASE_v1.4.0.md:33-35).

Parity: surogate/grpo/orchestrator/depth_controller.py:54-142.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, Dict, List, Optional


def _quantile(sorted_values: List[int], q: float) -> float:
    if not sorted_values:
        return 0.0
    pos = q * (len(sorted_values) - 1)
    lo = int(pos)
    hi = min(lo + 1, len(sorted_values) - 1)
    return sorted_values[lo] + (sorted_values[hi] - sorted_values[lo]) * (pos - lo)


@dataclass
class DepthObservation:
    depth: int           # turns the rollout took
    reward: float
    truncated: bool = False   # the cap ended it


class RolloutDepthController:
    def __init__(self, enabled: bool = True, quantile: float = 0.9, headroom: float = 1.25, min_cap: int = 2, max_cap: Optional[int] = None,
                 probe_every: int = 8, window: int = 512, min_observations: int = 32, reward_threshold: float = 0.0):
        self.enabled, self.q, self.headroom, self.min_cap, self.max_cap = enabled, quantile, headroom, min_cap, max_cap
        self.probe_every, self.min_obs, self.threshold = max(1, probe_every), min_observations, reward_threshold
        self.useful: Deque[int] = deque(maxlen=window)     # depths of rollouts that earned reward
        self._cap: Optional[int] = None
        self.truncated_rate = 0.0

    def is_probe_step(self, step: int) -> bool:
        return self.enabled and step % self.probe_every == 0

    def cap_for_step(self, step: int) -> Optional[int]:
        if not self.enabled or self.is_probe_step(step):
            return self.max_cap
        return self._cap if self._cap is not None else self.max_cap

    def observe(self, step: int, observations: List[DepthObservation]) -> None:
        if not observations:
            return
        self.truncated_rate = sum(o.truncated for o in observations) / len(observations)
        for o in observations:
            if o.reward > self.threshold and not o.truncated:
                self.useful.append(int(o.depth))
        if len(self.useful) >= self.min_obs:
            cap = int(_quantile(sorted(self.useful), self.q) * self.headroom + 0.999)
            cap = max(self.min_cap, cap)
            if self.max_cap is not None:
                cap = min(cap, self.max_cap)
            self._cap = cap

    @property
    def cap(self) -> Optional[int]:
        return self._cap

    def metrics(self) -> Dict[str, float]:
        return {"depth/cap": float(self._cap or 0), "depth/observations": float(len(self.useful)), "depth/truncated_rate": float(self.truncated_rate)}

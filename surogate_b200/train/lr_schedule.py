"""Learning-rate schedules: linear warm-up, then linear / cosine / constant / WSD, optional 1-sqrt cool-down,
plus a temporary override that blends back to the schedule and a permanent reduction (used by the loss guard).

Parity: surogate/train/lr_schedule.py:4-109.
"""
from __future__ import annotations

import math
from typing import Optional


def _one_minus_sqrt(hi: float, lo: float, frac: float) -> float:
    return lo + (hi - lo) * (1.0 - math.sqrt(min(max(frac, 0.0), 1.0)))


class LRSchedule:
    def __init__(self, base_lr: float, max_steps: int, warmup_steps: int = 0, cooldown_steps: int = 0, final_lr: float = 0.0,
                 schedule_type: str = "linear", wsd_decay_steps_fraction: float = 0.1):
        self.base_lr, self.final_lr = float(base_lr), float(final_lr)
        self.max_steps = int(max_steps)
        self.warmup = max(0, int(warmup_steps))
        self.cooldown = max(0, int(cooldown_steps))
        self.kind = schedule_type.lower()
        self.wsd_decay = max(0, int(self.max_steps * wsd_decay_steps_fraction))
        self.body = max(0, self.max_steps - self.warmup - self.cooldown)
        self._ovr: Optional[tuple] = None  # (lr, start_step, grace)

    def scheduled(self, step: int) -> float:
        if step < self.warmup:
            return self.base_lr * step / self.warmup
        cool_start = self.max_steps - self.cooldown
        if self.cooldown and step >= cool_start:
            return _one_minus_sqrt(self.base_lr, self.final_lr, (step - cool_start) / self.cooldown)
        if self.body == 0 or self.kind == "constant":
            return self.base_lr
        frac = min(1.0, (step - self.warmup) / self.body)
        if self.kind == "linear":
            return self.base_lr + (self.final_lr - self.base_lr) * frac
        if self.kind == "wsd":
            start = self.max_steps - self.wsd_decay
            if self.wsd_decay and step >= start:
                return _one_minus_sqrt(self.base_lr, self.final_lr, (step - start) / self.wsd_decay)
            return self.base_lr
        return self.final_lr + (self.base_lr - self.final_lr) * 0.5 * (1.0 + math.cos(math.pi * frac))  # cosine (default)

    def get_lr(self, step: int) -> float:
        lr = self.scheduled(step)
        if self._ovr is not None:
            o_lr, start, grace = self._ovr
            t = (step - start) / grace
            if t >= 1.0:
                self._ovr = None
            else:
                lr = o_lr + (lr - o_lr) * t
        return lr

    def override_lr(self, lr: float, step: int, grace_period: int) -> None:
        self._ovr = (float(lr), int(step), max(1, int(grace_period)))

    @property
    def has_override(self) -> bool:
        return self._ovr is not None

    def reduce_lr(self, factor: float) -> None:
        self.base_lr *= factor
        self.final_lr *= factor

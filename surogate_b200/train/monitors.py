"""Adaptive-training monitors fed once per step with (loss, grad-norm, MoE stats).

* LossGuard: spike / NaN detector that asks for a temporary or permanent LR cut.
* PlateauDetector: no relative improvement of the smoothed loss for N steps.
* PhaseDetector: labels the run (warmup / converging / plateau / unstable / diverging).
* GradientTracker: running statistics of the gradient norm and exploding/vanishing flags.
* MoEMonitor: routing-collapse and imbalance warnings from router statistics.
* EarlyStopping: stop on plateau with patience, or on divergence.
* TrainingAdvisor: turns the above into human-readable recommendations.

Parity: surogate/train/{loss_guard,plateau_detector,phase_detector,gradient_tracker,moe_monitor,
early_stopping,training_advisor}.py.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional


class _Ema:
    def __init__(self, beta: float):
        self.beta, self.v, self.n = beta, 0.0, 0

    def update(self, x: float) -> float:
        self.n += 1
        self.v = x if self.n == 1 else self.beta * self.v + (1 - self.beta) * x
        return self.v


@dataclass
class GuardAction:
    kind: str  # "none" | "override" | "reduce" | "abort"
    factor: float = 1.0
    grace: int = 0
    reason: str = ""


class LossGuard:
    def __init__(self, window: int = 50, spike_sigma: float = 4.0, spike_ratio: float = 1.5, max_strikes: int = 3, enabled: bool = True):
        self.hist: Deque[float] = deque(maxlen=window)
        self.sigma, self.ratio, self.max_strikes, self.enabled = spike_sigma, spike_ratio, max_strikes, enabled
        self.strikes = 0

    def check(self, loss: float, norm: float) -> GuardAction:
        if not self.enabled:
            return GuardAction("none")
        if not math.isfinite(loss) or not math.isfinite(norm):
            self.strikes += 1
            if self.strikes >= self.max_strikes:
                return GuardAction("abort", reason="repeated non-finite loss / gradient norm")
            return GuardAction("reduce", factor=0.5, reason="non-finite loss or gradient norm")
        act = GuardAction("none")
        if len(self.hist) >= 10:
            mean = sum(self.hist) / len(self.hist)
            var = sum((x - mean) ** 2 for x in self.hist) / len(self.hist)
            if loss > mean + self.sigma * math.sqrt(var) and loss > mean * self.ratio:
                self.strikes += 1
                act = (GuardAction("reduce", 0.5, reason=f"loss spike {loss:.3f} vs mean {mean:.3f} (strike {self.strikes})")
                       if self.strikes >= self.max_strikes else
                       GuardAction("override", 0.3, grace=50, reason=f"loss spike {loss:.3f} vs mean {mean:.3f}"))
                if act.kind == "reduce":
                    self.strikes = 0
                return act
        self.hist.append(loss)
        return act


class PlateauDetector:
    def __init__(self, patience: int = 200, min_rel_improvement: float = 1e-3, beta: float = 0.98):
        self.ema, self.best, self.since = _Ema(beta), math.inf, 0
        self.patience, self.tol = patience, min_rel_improvement

    def update(self, loss: float) -> bool:
        s = self.ema.update(loss)
        if s < self.best * (1 - self.tol):
            self.best, self.since = s, 0
        else:
            self.since += 1
        return self.since >= self.patience


class GradientTracker:
    def __init__(self, window: int = 100):
        self.hist: Deque[float] = deque(maxlen=window)

    def update(self, norm: float) -> Dict[str, float]:
        if math.isfinite(norm):
            self.hist.append(norm)
        n = max(1, len(self.hist))
        mean = sum(self.hist) / n
        std = math.sqrt(sum((x - mean) ** 2 for x in self.hist) / n)
        return {"mean": mean, "std": std, "max": max(self.hist, default=0.0), "exploding": float(norm > 10 * mean and n > 10),
                "vanishing": float(mean < 1e-7 and n > 10)}


class PhaseDetector:
    def __init__(self, warmup_steps: int = 0):
        self.warmup = warmup_steps
        self.fast, self.slow = _Ema(0.9), _Ema(0.99)
        self.noise = _Ema(0.95)

    def update(self, step: int, loss: float) -> str:
        if not math.isfinite(loss):
            return "diverging"
        f, s = self.fast.update(loss), self.slow.update(loss)
        n = self.noise.update(abs(loss - f))
        if step < self.warmup:
            return "warmup"
        if f > s * 1.2:
            return "diverging"
        if n > 0.15 * max(abs(f), 1e-8):
            return "unstable"
        if f < s * 0.995:
            return "converging"
        return "plateau"


class MoEMonitor:
    def __init__(self, imbalance_warn: float = 3.0, min_utilization: float = 0.5):
        self.imbalance_warn, self.min_util = imbalance_warn, min_utilization

    def check(self, stats: Dict[str, float]) -> List[str]:
        out = []
        if not stats:
            return out
        if stats.get("load_imbalance", 1.0) > self.imbalance_warn:
            out.append(f"expert load imbalance {stats['load_imbalance']:.2f}x: consider a larger router_aux_loss_coef")
        if stats.get("expert_utilization", 1.0) < self.min_util:
            out.append(f"only {100 * stats['expert_utilization']:.0f}% of experts receive tokens (routing collapse)")
        ent, mx = stats.get("router_entropy"), stats.get("router_entropy_max")
        if ent is not None and mx and ent < 0.3 * mx:
            out.append("router entropy is low: routing is close to deterministic")
        return out


class EarlyStopping:
    def __init__(self, enabled: bool = False, patience: int = 500):
        self.enabled = enabled
        self.plateau = PlateauDetector(patience=patience)

    def should_stop(self, loss: float, phase: str) -> bool:
        if not self.enabled:
            return False
        return self.plateau.update(loss) or phase == "diverging"


class TrainingAdvisor:
    def advise(self, phase: str, grad: Dict[str, float], moe_warnings: List[str]) -> List[str]:
        tips = list(moe_warnings)
        if phase == "unstable":
            tips.append("loss is noisy: lower the learning rate or raise gradient_accumulation_steps")
        if phase == "diverging":
            tips.append("loss is rising: lower the learning rate; check max_grad_norm and the warm-up length")
        if grad.get("exploding"):
            tips.append("gradient norm is an order of magnitude above its running mean")
        if grad.get("vanishing"):
            tips.append("gradient norm is vanishing: check loss masking and the learning-rate schedule")
        return tips

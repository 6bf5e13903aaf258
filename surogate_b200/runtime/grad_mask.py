"""Gradient masks for deliberate partial-update runs of a full (non-LoRA) model.

Two modes, chosen in the trainer config or by the environment variables the reference reads:

* ``allow_substrings`` (``SUROGATE_TRAINABLE_PARAM_SUBSTRINGS=a,b,...``): only parameters whose name contains one of the
  substrings (case-insensitive) train.  The others are frozen outright: no gradient buffer is written for them, they do
  not count in the gradient norm, and the optimizer leaves them (and their weight decay) alone.
* ``mlp_growth_new_half`` (``SUROGATE_GRADIENT_MASK_MODE=mlp_growth_new_half``): for a model whose MLP width was doubled,
  only the new half of every MLP matrix trains.  For the fused up/gate weight ``[2M, C]`` the first half of the rows of each of
  its two parts is zeroed in the gradient, for separate up / gate weights the first half of the rows, for the down weight
  ``[C, M]`` the first half of the columns.  Every other parameter is frozen, and weight decay is off for the MLP matrices
  because it would change their frozen half.

Parity: csrc/src/runtime/optimizers/gradient_mask.h (spec parsing :67-93, whole_param_trainable :118-138,
apply_partial_mask :140-184, weight_decay_for :186-194).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

_UP_OR_GATE = ("gate_proj", "up_proj", "mlp_gate_weight", "mlp_up_weight", "gate_weight", "up_weight")
_DOWN = ("down_proj", "mlp_down_weight", "down_weight")


def _has(name: str, needles: Sequence[str]) -> bool:
    n = name.lower()
    return any(x in n for x in needles)


@dataclass
class GradientMask:
    substrings: List[str] = field(default_factory=list)
    mlp_growth_new_half: bool = False

    @classmethod
    def resolve(cls, substrings: Optional[Sequence[str]] = None, mode: Optional[str] = None) -> Optional["GradientMask"]:
        """The mask from the explicit arguments, else from the environment; ``None`` when nothing asks for one."""
        if substrings is None:
            raw = os.environ.get("SUROGATE_TRAINABLE_PARAM_SUBSTRINGS", "")
            substrings = [s.strip() for s in raw.split(",") if s.strip()]
        if isinstance(substrings, str):
            substrings = [s.strip() for s in substrings.split(",") if s.strip()]
        mode = (mode if mode is not None else os.environ.get("SUROGATE_GRADIENT_MASK_MODE", "")).strip().lower()
        subs = [s.lower() for s in substrings]
        if mode in ("", "none", "off", "0"):
            return cls(subs) if subs else None
        if mode == "allow_substrings":
            if not subs:
                raise ValueError("gradient_mask_mode=allow_substrings needs trainable_param_substrings")
            return cls(subs)
        if mode == "mlp_growth_new_half":
            return cls(subs, mlp_growth_new_half=True)
        raise ValueError(f"unknown gradient mask mode '{mode}' (allow_substrings | mlp_growth_new_half)")

    # ------------------------------------------------------------------ name classes
    @staticmethod
    def is_mlp_up_or_gate(name: str) -> bool:
        return _has(name, ("mlp", "mixer")) and _has(name, _UP_OR_GATE)

    @staticmethod
    def is_mlp_down(name: str) -> bool:
        return _has(name, ("mlp", "mixer")) and _has(name, _DOWN)

    def is_growth_param(self, name: str) -> bool:
        return self.is_mlp_up_or_gate(name) or self.is_mlp_down(name)

    # ------------------------------------------------------------------ what the parameter store asks
    def trainable(self, name: str) -> bool:
        if self.substrings:
            return _has(name, self.substrings)
        if self.mlp_growth_new_half:
            return self.is_growth_param(name)
        return True

    def decays(self, name: str) -> bool:
        return not (self.mlp_growth_new_half and self.is_growth_param(name))

    def has_partial(self, name: str) -> bool:
        return self.mlp_growth_new_half and self.is_growth_param(name)

    def apply_partial(self, name: str, grad: torch.Tensor) -> None:
        """Zero the inherited half of an MLP matrix's gradient in place (``grad`` has the parameter's shape; a leading expert
        dimension is allowed)."""
        if not self.has_partial(name):
            return
        if grad.dim() < 2:
            raise ValueError(f"mlp_growth_new_half expects a matrix gradient for {name}, got shape {tuple(grad.shape)}")
        rows, cols = grad.shape[-2], grad.shape[-1]
        if self.is_mlp_up_or_gate(name):
            if "mlp_up_weight" in name.lower():  # fused [2M, C]: two parts of M rows, each with its old half first
                if rows % 4:
                    raise ValueError(f"mlp_growth_new_half expects a fused 2M row count for {name}, got {rows}")
                q = rows // 4
                grad[..., :q, :].zero_()
                grad[..., 2 * q:3 * q, :].zero_()
                return
            if rows % 2:
                raise ValueError(f"mlp_growth_new_half expects an even row count for {name}, got {rows}")
            grad[..., :rows // 2, :].zero_()
            return
        if cols % 2:
            raise ValueError(f"mlp_growth_new_half expects an even column count for {name}, got {cols}")
        grad[..., :, :cols // 2].zero_()

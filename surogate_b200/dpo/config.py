"""``surogate dpo`` configuration: the SFT key set plus the preference-optimisation knobs.

Parity: surogate/dpo/config.py.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..config.sft_config import SFTConfig


@dataclass
class DPOConfig(SFTConfig):
    beta: float = 0.1
    label_smoothing: float = 0.0
    loss_type: str = "sigmoid"  # sigmoid | ipo | hinge
    reference_free: bool = False
    max_prompt_length: int = 512
    sample_packing: bool = False
    learning_rate: float = 5e-6

    def finalize(self) -> None:
        super().finalize()
        if self.loss_type not in ("sigmoid", "ipo", "hinge"):
            raise ValueError(f"[E130] dpo loss_type must be sigmoid | ipo | hinge, got '{self.loss_type}'")
        if self.beta <= 0:
            raise ValueError("[E131] dpo beta must be positive")
        if not self.lora and not self.reference_free:
            raise ValueError("[E132] the frozen reference policy is the base model under LoRA: set lora: true or reference_free: true")

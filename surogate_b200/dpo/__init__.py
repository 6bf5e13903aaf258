"""Offline Direct Preference Optimisation on top of the trainer's objective hooks."""
from .config import DPOConfig  # noqa: F401
from .loss import dpo_loss_and_weights  # noqa: F401
from .trainer import DPOTrainer, dpo_main  # noqa: F401

"""Asynchronous GRPO reinforcement learning: orchestrator (rollouts, rewards, advantages), packer, transports, weight
broadcast and the trainer step built on the per-token gradient weights of the fused LM-head loss kernel."""
from .config import GRPOConfig  # noqa: F401
from .loss import grpo_token_weights, grpo_loss_reference  # noqa: F401

"""RL environments: a minimal environment / rubric interface and three built-in tasks."""
from .base import Environment, MultiTurnEnv, Rubric, SingleTurnEnv, as_reward_fn, evaluate, load_environment, openai_policy

__all__ = ["Environment", "MultiTurnEnv", "Rubric", "SingleTurnEnv", "as_reward_fn", "evaluate", "load_environment", "openai_policy"]

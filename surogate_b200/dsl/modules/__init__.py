"""Reusable DSL modules (attention, MLP, MoE, norms, embedding / LM head).

Parity: surogate/dsl/modules/*.py.
"""
from .core import Embedding, LMHead, RMSNorm, Linear
from .attention import GenericGQAttention, AttentionConfig
from .mlp import GenericMLP, MLPConfig
from .moe import MoEExpertsGated, MoESharedExpert

__all__ = ["Embedding", "LMHead", "RMSNorm", "Linear", "GenericGQAttention", "AttentionConfig", "GenericMLP",
           "MLPConfig", "MoEExpertsGated", "MoESharedExpert"]

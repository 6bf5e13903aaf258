"""Optimizers operating on the flat per-bucket shards of the parameter store.

Parity: csrc/src/runtime/optimizers/ (adamw.cu, flash_adamw_8bit.cu, normuon.cu, polar_express.cu, cpu_adamw.cpp).
"""
from .adamw import AdamW, AdamW8bit, OptimizerConfig, make_optimizer
from .normuon import NorMuon

__all__ = ["AdamW", "AdamW8bit", "NorMuon", "OptimizerConfig", "make_optimizer"]

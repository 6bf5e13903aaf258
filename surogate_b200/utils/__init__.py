"""Utilities: logging, system/GPU info, MoE statistics, speed-of-light model, adapter merge."""

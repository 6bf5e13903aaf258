"""Checkpoint I/O: HF safetensors import/export, sharded step checkpoints, PEFT adapters, token shard files."""

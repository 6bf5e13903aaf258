"""A rough memory estimate of a run, shown next to each GPU as "fits / tight / risk" while a launch is put together.

The estimate is deliberately coarse (a guide for choosing a GPU, not a guarantee): parameter count from the model's name
(``Qwen3-8B`` -> 8; a mixture-of-experts name such as ``30B-A3B`` has 30 B stored and 3 B active), weight bytes by recipe (LoRA
keeps the base frozen and may store it quantised), optimizer state by optimizer, activations by tokens per micro-batch with or
without recomputation, ZeRO sharding over the GPUs of the run.  The trainer's own static buffer plan (``Trainer.activation_plan``)
is the exact counterpart once a model is built.

Parity: jackalope/src/launch.ts (paramsBFromModel, estimateRunVramGB, fitOnGpu).
"""
from __future__ import annotations

import re
from typing import Optional, Tuple

RECIPE_WEIGHT_BYTES = {"bf16": 2.0, "fp8-hybrid": 2.0, "fp8_hybrid": 2.0, "nvfp4": 2.0, "nvfp4_quartet": 2.0}  # master copies stay bf16
QLORA_WEIGHT_BYTES = {"none": 2.0, "fp8": 1.0, "bnb": 0.56, "nf4": 0.56, "fp4": 0.56, "nvfp4": 0.56, "mxfp4": 0.53}
OPTIMIZER_STATE_BYTES = {"adamw": 8.0, "adamw_8bit": 2.1, "normuon": 2.0}


def params_billions(model: str) -> Optional[Tuple[float, float]]:
    """(stored, active) parameter counts in billions parsed from a model id, or None when the name carries no count."""
    name = model.rsplit("/", 1)[-1]
    sizes = re.findall(r"(?<![A-Za-z0-9.])(\d+(?:\.\d+)?)\s*[Bb](?![A-Za-z])", name)
    active = re.search(r"(?<![A-Za-z0-9])A(\d+(?:\.\d+)?)[Bb](?![A-Za-z])", name)
    if not sizes and not active:
        m = re.search(r"(\d+(?:\.\d+)?)\s*[Mm](?![A-Za-z])", name)
        if not m:
            return None
        v = float(m.group(1)) / 1000.0
        return v, v
    total = float(sizes[0]) if sizes else float(active.group(1))
    return total, float(active.group(1)) if active else total


def estimate_run_memory_gb(model: str, recipe: str = "bf16", lora: bool = True, qlora: str = "none", optimizer: str = "adamw_8bit",
                           per_device_batch: int = 2, sequence_len: int = 2048, recompute: bool = True, gpus: int = 1,
                           zero_level: int = 1) -> Optional[float]:
    """GB per GPU, or None when the parameter count is unknown."""
    p = params_billions(model)
    if p is None:
        return None
    total, active = p
    gpus = max(1, gpus)
    if lora:
        weights = total * QLORA_WEIGHT_BYTES.get(qlora, 2.0)
        trainable = total * 0.01
        state = trainable * (2.0 + 4.0 + OPTIMIZER_STATE_BYTES.get(optimizer, 8.0))  # adapter + fp32 gradient + moments
    else:
        shard_w = gpus if zero_level >= 3 else 1
        shard_g = gpus if zero_level >= 2 else 1
        shard_o = gpus if zero_level >= 1 else 1
        weights = total * RECIPE_WEIGHT_BYTES.get(recipe, 2.0) / shard_w
        if recipe != "bf16":
            weights += min(total, 2.0 * active) * 1.0 / shard_w  # quantised working copies of the layers in flight
        state = total * 4.0 / shard_g + total * OPTIMIZER_STATE_BYTES.get(optimizer, 8.0) / shard_o
    tokens = max(1, per_device_batch) * max(1, sequence_len)
    act_per_token_gb = active * (0.012 if recompute else 0.10) / 1024.0  # saved residuals only vs every saved activation
    activations = tokens * act_per_token_gb * 8.0 / max(1.0, active ** 0.5)
    return round(weights + state + activations + 1.5, 1)  # + context, workspaces, allocator slack


def fit_verdict(estimate_gb: Optional[float], free_gb: Optional[float]) -> str:
    if estimate_gb is None or free_gb is None:
        return "unknown"
    if free_gb >= 1.3 * estimate_gb:
        return "fits"
    return "tight" if free_gb >= estimate_gb else "risk"

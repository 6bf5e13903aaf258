"""Exploration noise on the rollout engine's normalisation weights (adaptive quantisation noise, QeRL).

Between the trainer and the inference engine the published weights may carry Gaussian noise on their RMSNorm scale vectors:
multiplying a norm weight by (1 + eps) perturbs every downstream projection the way quantisation noise would, which raises the
sampling entropy early in training.  The standard deviation follows a staged schedule: no noise during the first stage, then
``sigma_start`` decaying geometrically to ``sigma_end`` over the remaining ``stages - 1`` stages.  The noise is applied to a
PUBLISHED copy only (a directory of safetensors files); the trainer's own weights never see it.  The sigma in force is written to
``noise_sigma.json`` next to the files so that an engine which applies the noise itself (adapters: the base model's norms are
not in the adapter) can read it.

Parity: surogate/grpo/noise_scheduler.py (compute_sigma, inject_noise_into_safetensors, write_noise_sigma).
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass
from typing import Dict, Optional

import torch

NORM_WEIGHT = re.compile(r"(layernorm|_norm|\.norm|norm_f)\.weight$")
SIGMA_FILE = "noise_sigma.json"


@dataclass
class NoiseConfig:
    enabled: bool = False
    sigma_start: float = 1e-2
    sigma_end: float = 1e-4
    stages: int = 10
    seed: int = 0


def sigma_at(step: int, total_steps: int, cfg: NoiseConfig) -> float:
    if not cfg.enabled or total_steps <= 0 or cfg.stages < 2:
        return 0.0
    stage = min(cfg.stages - 1, int(min(step, total_steps - 1) * cfg.stages // total_steps))
    if stage == 0:
        return 0.0
    if cfg.stages == 2:
        return float(cfg.sigma_start)
    frac = (stage - 1) / (cfg.stages - 2)
    return float(cfg.sigma_start * (cfg.sigma_end / cfg.sigma_start) ** frac)


def add_noise_to_directory(directory: str, sigma: float, seed: int = 0) -> int:
    """Adds N(0, sigma^2) to every normalisation weight of every safetensors file under ``directory`` (in place, dtype kept) and
    records sigma.  Returns how many tensors were changed."""
    from safetensors.torch import load_file, save_file

    changed = 0
    gen = torch.Generator().manual_seed(seed)
    if sigma > 0:
        for fn in sorted(os.listdir(directory)):
            if not fn.endswith(".safetensors"):
                continue
            path = os.path.join(directory, fn)
            tensors = load_file(path)
            touched = False
            for name in sorted(tensors):
                if NORM_WEIGHT.search(name) and tensors[name].dim() == 1:
                    t = tensors[name]
                    tensors[name] = (t.float() + sigma * torch.randn(t.shape, generator=gen)).to(t.dtype)
                    changed += 1
                    touched = True
            if touched:
                save_file(tensors, path + ".tmp", metadata={"format": "pt"})
                os.replace(path + ".tmp", path)
    with open(os.path.join(directory, SIGMA_FILE), "w") as f:
        json.dump({"sigma": sigma, "tensors_changed": changed}, f)
    return changed


def read_sigma(directory: str) -> Optional[Dict[str, float]]:
    try:
        with open(os.path.join(directory, SIGMA_FILE)) as f:
            return json.load(f)
    except FileNotFoundError:
        return None

"""RoPE frequency tables with the scaling variants found in HF ``config.json`` files.

``rope_inv_freq(rotary_dim, theta, scaling)`` returns ``(inv_freq [rotary_dim/2], attention_factor)``; ``scaling`` is the
HF ``rope_scaling`` / ``rope_parameters`` dict (``rope_type`` or legacy ``type``): default, linear, dynamic (NTK, evaluated
at ``max_position_embeddings``), yarn, llama3.  cos / sin are multiplied by ``attention_factor`` (YaRN's mscale).

Parity: csrc/src/config/rope_config.h (linear / dynamic / yarn / llama3 scaling).
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch


def _yarn_find_dim(num_rot: float, dim: int, base: float, max_pos: int) -> float:
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def rope_inv_freq(rotary_dim: int, theta: float, scaling: Optional[Dict[str, Any]] = None, max_position_embeddings: Optional[int] = None,
                  device=None) -> Tuple[torch.Tensor, float]:
    idx = torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=device)
    inv = 1.0 / (theta ** (idx / rotary_dim))
    if not scaling:
        return inv, 1.0
    kind = (scaling.get("rope_type") or scaling.get("type") or "default").lower()
    factor = float(scaling.get("factor", 1.0))
    if kind == "default":
        return inv, 1.0
    if kind == "linear":
        return inv / factor, 1.0
    if kind == "dynamic":
        orig = int(scaling.get("original_max_position_embeddings") or max_position_embeddings or 0)
        seq = int(max_position_embeddings or orig)
        if orig and seq > orig:
            base = theta * ((factor * seq / orig) - (factor - 1)) ** (rotary_dim / (rotary_dim - 2))
            inv = 1.0 / (base ** (idx / rotary_dim))
        return inv, 1.0
    if kind == "llama3":
        lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv
        scaled = torch.where(wavelen > old / lo, inv / factor, inv)
        smooth = (old / wavelen - lo) / (hi - lo)
        mid = (1 - smooth) * inv / factor + smooth * inv
        is_mid = (wavelen <= old / lo) & (wavelen >= old / hi)
        return torch.where(is_mid, mid, scaled), 1.0
    if kind == "proportional":
        # only the first fraction of the frequency pairs rotates; the rest get angle 0 (identity), and the exponent's
        # denominator stays the full head size, so the rotated pairs keep the frequencies they would have in a full rotation
        angles = int(float(scaling.get("partial_rotary_factor", 1.0)) * rotary_dim // 2)
        rot = 1.0 / (theta ** (torch.arange(0, 2 * angles, 2, dtype=torch.float32, device=device) / rotary_dim))
        return torch.cat([rot, torch.zeros(rotary_dim // 2 - angles, dtype=torch.float32, device=device)]) / factor, 1.0
    if kind == "yarn":
        orig = int(scaling.get("original_max_position_embeddings") or max_position_embeddings or 4096)
        beta_fast, beta_slow = float(scaling.get("beta_fast", 32.0)), float(scaling.get("beta_slow", 1.0))
        mscale, mscale_all = scaling.get("mscale"), scaling.get("mscale_all_dim")

        def get_mscale(scale, m=1.0):
            return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

        if scaling.get("attention_factor") is not None:
            att = float(scaling["attention_factor"])
        elif mscale and mscale_all:
            att = get_mscale(factor, mscale) / get_mscale(factor, mscale_all)
        else:
            att = get_mscale(factor)
        low = _yarn_find_dim(beta_fast, rotary_dim, theta, orig)
        high = _yarn_find_dim(beta_slow, rotary_dim, theta, orig)
        if scaling.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, rotary_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(rotary_dim // 2, dtype=torch.float32, device=device) - low) / (high - low)).clamp(0, 1)
        extrap = 1 - ramp
        return (inv / factor) * (1 - extrap) + inv * extrap, att
    raise ValueError(f"[E150] unsupported rope scaling type '{kind}'")

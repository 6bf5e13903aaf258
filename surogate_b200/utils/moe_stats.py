"""Router statistics summarised per step (utilisation, imbalance, entropy ...).

Parity: csrc/src/kernels/moe/moe_diagnostics.cu + IRunState MoE stats tuple (runtime/training/model.h:418-431).
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch


def summarize(stats: List[Tuple[int, torch.Tensor, torch.Tensor]]) -> Dict[str, float]:
    """``stats`` = [(layer, tokens-per-expert counts [E], mean router probability [E])]."""
    if not stats:
        return {}
    counts = torch.stack([c.float() for _, c, _ in stats])  # [layers, E]
    probs = torch.stack([p.float() for _, _, p in stats])
    frac = counts / counts.sum(1, keepdim=True).clamp_min(1)
    E = counts.shape[1]
    mean = frac.mean(1, keepdim=True)
    ent = -(probs.clamp_min(1e-20) * probs.clamp_min(1e-20).log()).sum(1)
    return {
        "num_layers": float(counts.shape[0]),
        "expert_utilization": float((counts > 0).float().mean()),
        "active_experts": float((counts > 0).float().sum(1).mean()),
        "dead_experts": float((counts == 0).float().sum(1).mean()),   # experts that received no token, per layer on average
        "load_imbalance": float((frac.max(1).values / mean.squeeze(1)).mean()),
        "max_fraction": float(frac.max()),
        "min_fraction": float(frac.min()),
        "load_cv": float((frac.std(1) / mean.squeeze(1)).mean()),
        "router_entropy": float(ent.mean()),
        "router_entropy_max": float(torch.log(torch.tensor(float(E)))),
    }

"""Stage planner for dispatch-PP (pipeline-like layer dispatch for GPUs without a fast interconnect).

Layers are cut into small stages of ``stage_layers`` blocks (default 4), at least as many stages as GPUs; stage ``s`` runs
on GPU ``s % gpus``.  ``M = gpus * grad_accum`` micro-batches travel through the stages in a diagonal wavefront: at tick
``t`` stage ``s`` processes micro-batch ``t - s`` (forward), and the backward wave runs the same diagonal in reverse.
``wavefront`` returns that schedule; ``parallel/dispatch_pp.py`` (PipelineTrainer) executes it.

Parity: surogate/train/dispatch_pp.py:22-54, docs/guides/dispatch-pp.md.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple


@dataclass
class Stage:
    index: int
    first_layer: int
    last_layer: int  # exclusive
    gpu: int

    @property
    def layers(self) -> range:
        return range(self.first_layer, self.last_layer)


def plan_stages(n_layers: int, gpus: int, stage_layers: int = 4, align: int = 1) -> List[Stage]:
    if n_layers < 1 or gpus < 1:
        raise ValueError("n_layers and gpus must be positive")
    size = max(1, min(stage_layers, n_layers // gpus if n_layers >= gpus else 1))
    if align > 1:
        size = max(align, size // align * align)
    n_stages = max(min(gpus, n_layers), -(-n_layers // size))
    # spread the remainder so stage sizes differ by at most one aligned unit
    base, extra = divmod(n_layers, n_stages)
    stages, at = [], 0
    for s in range(n_stages):
        n = base + (1 if s < extra else 0)
        stages.append(Stage(s, at, at + n, s % gpus))
        at += n
    return stages


def wavefront(n_stages: int, n_micro: int) -> List[List[Tuple[str, int, int]]]:
    """Ticks of (phase, stage, micro_batch).  Forward diagonal first, then the backward diagonal (last stage first)."""
    ticks: List[List[Tuple[str, int, int]]] = []
    for t in range(n_stages + n_micro - 1):
        ticks.append([("fwd", s, t - s) for s in range(n_stages) if 0 <= t - s < n_micro])
    for t in range(n_stages + n_micro - 1):
        ticks.append([("bwd", s, t - (n_stages - 1 - s)) for s in reversed(range(n_stages)) if 0 <= t - (n_stages - 1 - s) < n_micro])
    return ticks

"""The artifact any training run writes when ``SUROGATE_REGRESSION_ARTIFACT=<path>`` is set: the convergence curve (step, loss,
gradient norm, learning rate), step-time percentiles, peak device memory and the graph compiler's buffer-plan summary, so that a
harness can launch real configs as subprocesses and compare what comes back (``compare_runs``).

Parity: surogate/train/trainer.py:289-292, :841-915 (the same top-level keys and ``schema_version``);
surogate/regression/baseline_runner.py:311 (the harness sets the variable per run).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

ENV = "SUROGATE_REGRESSION_ARTIFACT"


def percentile_summary(values: List[float]) -> Dict[str, float]:
    if not values:
        return {}
    v = sorted(values)

    def q(f: float) -> float:
        return v[min(len(v) - 1, int(f * len(v)))]

    return {"count": float(len(v)), "min": v[0], "p50": q(0.5), "p90": q(0.9), "p95": q(0.95), "max": v[-1], "mean": sum(v) / len(v)}


class RunArtifact:
    def __init__(self, path: str):
        self.path = path
        self.curve: List[Dict[str, float]] = []
        self.step_ms: List[float] = []
        self.peak_bytes: Optional[int] = None

    @classmethod
    def from_env(cls, environ=os.environ) -> Optional["RunArtifact"]:
        p = environ.get(ENV)
        return cls(p) if p else None

    def add(self, step: int, loss: float, norm: float, lr: float, ms: float, peak_bytes: Optional[int] = None) -> None:
        self.curve.append({"step": float(step), "loss": float(loss), "grad_norm": float(norm), "lr": float(lr)})
        self.step_ms.append(float(ms))
        if peak_bytes is not None:
            self.peak_bytes = max(self.peak_bytes or 0, int(peak_bytes))

    def payload(self, trainer=None) -> Dict[str, Any]:
        plan: Dict[str, Any] = {}
        store: Dict[str, Any] = {}
        if trainer is not None:
            try:
                p = trainer.activation_plan()
                plan = {"saved_bytes": int(p.saved_bytes), "temp_bytes": int(p.temp_bytes),
                        **{f"{bt}.{ph}.tensors": len(pp.tensors) for bt, phases in p.per_block.items() for ph, pp in phases.items()}}
            except Exception:  # noqa: BLE001 - a model whose graphs the planner does not cover: the artifact goes without
                plan = {}
            try:
                store = {"buckets": len(trainer.store.buckets), "num_parameters": int(trainer.num_parameters())}
            except Exception:  # noqa: BLE001
                store = {}
        return {"schema_version": 1, "activation_snapshots": {}, "gradient_snapshots": {}, "convergence_curve": self.curve,
                "step_time_ms": percentile_summary(self.step_ms[1:] or self.step_ms),  # the first step pays one-time costs
                "cuda_peak_memory_bytes": self.peak_bytes, "nccl": {}, "descriptor_summary": store, "block_schema_summary": {},
                "buffer_plan_summary": plan}

    def write(self, trainer=None) -> str:
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(self.payload(trainer), f, indent=1)
        os.replace(tmp, self.path)
        return self.path


def compare_runs(new: Dict[str, Any], base: Dict[str, Any], loss_rtol: float = 2e-2, time_factor: float = 1.5, mem_factor: float = 1.15) -> List[str]:
    """Problems of ``new`` against ``base`` (both artifacts of this schema); empty when the run matches."""
    problems: List[str] = []
    a, b = new.get("convergence_curve") or [], base.get("convergence_curve") or []
    if len(a) != len(b):
        problems.append(f"step count {len(a)} != {len(b)}")
    for x, y in zip(a, b):
        if abs(x["loss"] - y["loss"]) > loss_rtol * max(abs(y["loss"]), 1e-6):
            problems.append(f"loss at step {int(y['step'])}: {x['loss']:.5f} vs baseline {y['loss']:.5f}")
            break
    ta, tb = (new.get("step_time_ms") or {}).get("p50"), (base.get("step_time_ms") or {}).get("p50")
    if ta and tb and ta > time_factor * tb:
        problems.append(f"step time p50 {ta:.1f} ms > {time_factor}x baseline {tb:.1f} ms")
    ma, mb = new.get("cuda_peak_memory_bytes"), base.get("cuda_peak_memory_bytes")
    if ma and mb and ma > mem_factor * mb:
        problems.append(f"peak memory {ma} > {mem_factor}x baseline {mb}")
    for key in ("descriptor_summary", "buffer_plan_summary"):
        if base.get(key) and new.get(key) and {k: v for k, v in new[key].items() if k != "temp_bytes"} != {k: v for k, v in base[key].items() if k != "temp_bytes"}:
            problems.append(f"{key} changed: {new[key]} vs {base[key]}")
    return problems

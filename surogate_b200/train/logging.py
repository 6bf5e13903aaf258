"""Run logger: JSON-lines file + console line per step, plus the JSONL metrics feed a dashboard can tail.

Console format (fields separated by ' | '):
``:: step   12 [ 4.0%] loss 2.3456 | norm 0.98 | 123.4k tps | 412 ms | sol 41.2% | eta 0:12:03 | phase converging``
JSON record: ``{"log":"step","time":...,"step":..,"epoch":..,"step_tokens":..,"duration_ms":..,"norm":..,"loss":..,"lr":..}``.
tokens/s is ``1000 * step_tokens / duration_ms`` with ``step_tokens = B * T * grad_accum * gpus``.

Parity: csrc/src/runtime/training/logging.cpp:278-381, docs/guides/metrics.md, surogate/train/metrics_writer.py.
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Any, Dict, Optional


def _fmt_tps(tps: float) -> str:
    return f"{tps / 1e3:.1f}k" if tps >= 1e3 else f"{tps:.0f}"


def _fmt_eta(seconds: float) -> str:
    seconds = int(max(0, seconds))
    return f"{seconds // 3600}:{seconds % 3600 // 60:02d}:{seconds % 60:02d}"


class TrainingRunLogger:
    def __init__(self, log_file: Optional[str] = None, metrics_path: Optional[str] = None, is_main: bool = True, stream=None):
        self.is_main = is_main
        self.stream = stream or sys.stdout
        self.f = None
        self.metrics = None
        if is_main and log_file:
            os.makedirs(os.path.dirname(os.path.abspath(log_file)), exist_ok=True)
            self.f = open(log_file, "a")
        if is_main and metrics_path:
            try:
                self.metrics = open(metrics_path, "a")
            except OSError:
                self.metrics = None
        self.t_start = time.time()

    def _write(self, rec: Dict[str, Any]) -> None:
        rec = {"time": time.time(), **rec}
        line = json.dumps(rec, default=str)
        if self.f:
            self.f.write(line + "\n")
            self.f.flush()
        if self.metrics and rec.get("log") in ("step", "eval", "gpu", "moe"):
            self.metrics.write(line + "\n")
            self.metrics.flush()

    def log_step(self, step: int, max_steps: int, epoch: float, loss: float, norm: float, lr: float, step_tokens: int, duration_ms: float,
                 sol: Optional[float] = None, phase: Optional[str] = None, extra: Optional[Dict[str, Any]] = None) -> str:
        tps = 1000.0 * step_tokens / max(duration_ms, 1e-9)
        pct = 100.0 * step / max(1, max_steps)
        eta = (max_steps - step) * duration_ms / 1e3
        parts = [f":: step {step:5d} [{pct:5.1f}%] loss {loss:.4f}", f"norm {norm:.3f}", f"{_fmt_tps(tps)} tps", f"{duration_ms:.0f} ms"]
        if sol is not None:
            parts.append(f"sol {100 * sol:.1f}%")
        parts.append(f"eta {_fmt_eta(eta)}")
        if phase:
            parts.append(f"phase {phase}")
        line = " | ".join(parts)
        if self.is_main:
            print(line, file=self.stream, flush=True)
            self._write({"log": "step", "step": step, "epoch": epoch, "step_tokens": step_tokens, "duration_ms": duration_ms, "norm": norm,
                         "loss": loss, "lr": lr, "tps": tps, "sol": sol, "phase": phase, **(extra or {})})
        return line

    def log_eval(self, step: int, loss: float, duration_ms: float = 0.0) -> None:
        if self.is_main:
            print(f":: eval  {step:5d} loss {loss:.4f}", file=self.stream, flush=True)
            self._write({"log": "eval", "step": step, "loss": loss, "duration_ms": duration_ms})

    def log_record(self, kind: str, **fields) -> None:
        """kinds: moe, gpu, allocator, dataset, options, sol, message."""
        if self.is_main:
            self._write({"log": kind, **fields})

    def message(self, text: str) -> None:
        if self.is_main:
            print(text, file=self.stream, flush=True)
            self._write({"log": "message", "text": text})

    def close(self) -> None:
        for f in (self.f, self.metrics):
            if f:
                f.close()
        self.f = self.metrics = None

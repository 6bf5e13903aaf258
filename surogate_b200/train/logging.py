"""Run logger: JSON-lines file + console line per step, plus the JSONL metrics feed a dashboard can tail.

Console format (fields separated by ' | '):
``:: step   12 [ 4.0%] loss 2.3456 | norm 0.98 | 123.4k tps | 412 ms | sol 41.2% | eta 0:12:03 | phase converging``
JSON record: ``{"log":"step","time":...,"step":..,"epoch":..,"step_tokens":..,"duration_ms":..,"norm":..,"loss":..,"lr":..}``.
tokens/s is ``1000 * step_tokens / duration_ms`` with ``step_tokens = B * T * grad_accum * gpus``.

The metrics feed (``report_to: [surogate]``) uses the dashboard's record schema, so a dashboard written for it reads the feed
unchanged: a step is ``{"step", "ts", "train/loss", "train/norm", "train/lr", "train/epoch", "train/tokens_per_second",
"train/phase", ...}``, an evaluation ``{"step", "ts", "eval/loss", ...}``, the run's options ``{"type": "config", "ts", ...scalars}``,
GPU telemetry ``{"type": "gpu", "step", "gpu_id", "ts", "temperature", "power", "gpu_utilization", "mem_utilization", ...}``; MoE
statistics go out as ``{"type": "moe", ...}`` (readers of the dashboard schema skip types they do not know).  The feed path is the
config's ``surogate_metrics_path``, or the environment variable ``SUROGATE_METRICS_PATH`` when the config leaves the default.

Parity: csrc/src/runtime/training/logging.cpp:278-381, docs/guides/metrics.md, surogate/train/metrics_writer.py,
surogate/train/reporter.py:284-330 (log line -> feed record).
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Any, Dict, Optional


DEFAULT_METRICS_PATH = "/tmp/surogate_metrics.jsonl"
ENV_METRICS_PATH = "SUROGATE_METRICS_PATH"


def resolve_metrics_path(configured: Optional[str]) -> str:
    """The feed path: an explicit config value wins, then the environment variable (how a launcher points a run at its own
    feed file without editing the config), then the default."""
    if configured and configured != DEFAULT_METRICS_PATH:
        return configured
    return os.environ.get(ENV_METRICS_PATH) or configured or DEFAULT_METRICS_PATH


def _scalars(d: Dict[str, Any], skip=()) -> Dict[str, Any]:
    return {k: v for k, v in d.items() if k not in skip and isinstance(v, (int, float)) and not isinstance(v, bool)}


def feed_record(rec: Dict[str, Any]) -> Optional[Dict[str, Any]]:
    """One log record (``{"log": kind, ...}``) as the feed record a dashboard reads, or None for kinds the feed does not carry."""
    kind, ts = rec.get("log"), rec.get("time", time.time())
    if kind == "step":
        out = {"step": rec.get("step", 0), "ts": ts}
        out.update({f"train/{k}": v for k, v in _scalars(rec, ("log", "step", "time", "step_tokens", "tps", "max_steps")).items()})
        if rec.get("duration_ms"):
            out["train/tokens_per_second"] = rec.get("step_tokens", 0) / (rec["duration_ms"] / 1000.0)
        elif isinstance(rec.get("tps"), (int, float)):
            out["train/tokens_per_second"] = rec["tps"]
        if rec.get("phase"):
            out["train/phase"] = rec["phase"]
        if rec.get("max_steps"):
            out["max_steps"] = rec["max_steps"]
        return out
    if kind == "eval":
        out = {"step": rec.get("step", 0), "ts": ts}
        out.update({f"eval/{k}": v for k, v in _scalars(rec, ("log", "step", "time", "eval_tokens")).items()})
        if rec.get("duration_ms") and rec.get("eval_tokens"):
            out["eval/tokens_per_second"] = rec["eval_tokens"] / (rec["duration_ms"] / 1000.0)
        return out
    if kind == "gpu":
        out = {"type": "gpu", "step": rec.get("step", 0), "gpu_id": rec.get("id", rec.get("index", 0)), "ts": ts}
        if isinstance(rec.get("name"), str):
            out["name"] = rec["name"]
        out.update(_scalars(rec, ("log", "step", "time", "id", "index", "throttle_reasons")))
        # the names the dashboard reads, next to this framework's own
        for theirs, ours in (("temperature", "temperature_c"), ("power", "power_w"), ("gpu_utilization", "gpu_util"), ("mem_utilization", "mem_util")):
            if ours in rec and theirs not in out:
                out[theirs] = rec[ours]
        return out
    if kind == "moe":
        return {"type": "moe", "ts": ts, **{k: v for k, v in rec.items() if k not in ("log", "time")}}
    if kind == "options":
        cfg = rec.get("config") or {}
        flat = {k: v for k, v in cfg.items() if isinstance(v, (str, int, float, bool)) or v is None}
        flat.setdefault("model", cfg.get("model") if isinstance(cfg.get("model"), str) else None)
        return {"type": "config", "ts": ts, **flat}
    return None


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
        if self.metrics:
            fr = feed_record(rec)
            if fr is not None:
                self.metrics.write(json.dumps(fr, default=str) + "\n")
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
            self._write({"log": "step", "step": step, "max_steps": max_steps, "epoch": epoch, "step_tokens": step_tokens, "duration_ms": duration_ms, "norm": norm,
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

"""Experiment reporters: Weights & Biases, Aim and the JSONL feed the terminal dashboard tails.

``make_reporters(cfg)`` builds one reporter per entry of ``report_to``; a reporter whose package is missing warns once
and turns itself off instead of failing the run.

Parity: surogate/train/reporter.py, metrics_writer.py:9.
"""
from __future__ import annotations

import json
import os
import time
import warnings
from typing import Any, Dict, List, Optional


class Reporter:
    name = "base"

    def log(self, step: int, metrics: Dict[str, Any]) -> None:
        pass

    def log_config(self, config: Dict[str, Any]) -> None:
        pass

    def finish(self) -> None:
        pass


class JsonlReporter(Reporter):
    """Append-only JSONL (default /tmp/surogate_metrics.jsonl): one record per step, eval, gpu and moe event."""
    name = "surogate"

    def __init__(self, path: str, run_name: str = ""):
        self.path, self.run = path, run_name
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self.f = open(path, "a")

    def log(self, step: int, metrics: Dict[str, Any]) -> None:
        from .logging import feed_record

        rec = {"time": time.time(), "run": self.run, "step": step, **metrics}
        rec = feed_record(rec) if "log" in rec else rec  # log records go out in the dashboard's schema, anything else as it is
        if rec is not None:
            self.f.write(json.dumps(rec, default=str) + "\n")
            self.f.flush()

    def log_config(self, config: Dict[str, Any]) -> None:
        self.log(0, {"log": "options", "config": config})

    def finish(self) -> None:
        self.f.close()


class WandbReporter(Reporter):
    name = "wandb"

    def __init__(self, project: str, run_name: str, config: Optional[Dict[str, Any]] = None):
        import wandb  # type: ignore

        self.wandb = wandb
        self.run = wandb.init(project=project, name=run_name, config=config or {}, reinit=True)

    def log(self, step: int, metrics: Dict[str, Any]) -> None:
        self.wandb.log({k: v for k, v in metrics.items() if isinstance(v, (int, float))}, step=step)

    def finish(self) -> None:
        self.run.finish()


class AimReporter(Reporter):
    name = "aim"

    def __init__(self, experiment: str, run_name: str, config: Optional[Dict[str, Any]] = None, repo: Optional[str] = None):
        from aim import Run  # type: ignore

        self.run = Run(experiment=experiment, **({"repo": repo} if repo else {}))
        self.run.name = run_name
        if config:
            self.run["hparams"] = config

    def log(self, step: int, metrics: Dict[str, Any]) -> None:
        for k, v in metrics.items():
            if isinstance(v, (int, float)):
                self.run.track(v, name=k, step=step)

    def finish(self) -> None:
        self.run.close()


def make_reporters(report_to: List[str], run_name: str, project: str = "Surogate", metrics_path: str = "/tmp/surogate_metrics.jsonl",
                   config: Optional[Dict[str, Any]] = None) -> List[Reporter]:
    """``config`` (the run's options) also carries the reporters' own keys: ``wandb_project`` / ``wandb_name``, ``aim_experiment`` /
    ``aim_repo`` / ``aim_name``; each falls back to ``project`` / ``run_name``."""
    out: List[Reporter] = []
    c = config or {}
    for name in report_to or []:
        try:
            if name == "wandb":
                out.append(WandbReporter(c.get("wandb_project") or project, c.get("wandb_name") or run_name, config))
            elif name == "aim":
                out.append(AimReporter(c.get("aim_experiment") or project, c.get("aim_name") or run_name, config, c.get("aim_repo")))
            elif name in ("surogate", "jsonl"):
                out.append(JsonlReporter(metrics_path, run_name))
            else:
                warnings.warn(f"unknown reporter '{name}' (wandb | aim | surogate)")
        except ImportError:
            warnings.warn(f"report_to: '{name}' is not installed; reporting to it is disabled")
    return out

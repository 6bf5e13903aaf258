"""Run isolation: each launched run owns ``<root>/<stamp>-<label>/`` with

    metrics.jsonl       the feed the monitor tails
    metrics.jsonl.pid   {"pid", "start"} of a local run (stop / liveness)
    config.yaml         the exact config the run was started with
    train.log           the run's standard output and error
    meta.json           mode, model, dataset, recipe, GPUs, where it runs
    output/             checkpoints and the final model (``output_dir``), or what ``fetch`` brought back

so concurrent runs never interleave and the history is comparable.  The root is ``~/.surogate-watch/runs`` unless
``SUROGATE_RUNS_DIR`` names another.

Parity: jackalope/src/runs.ts.
"""
from __future__ import annotations

import json
import os
import re
import time
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from .records import parse_feed_line


def runs_root(root: Optional[str] = None) -> str:
    return root or os.environ.get("SUROGATE_RUNS_DIR") or os.path.join(os.path.expanduser("~"), ".surogate-watch", "runs")


def slug(text: str, limit: int = 40) -> str:
    return re.sub(r"[^a-zA-Z0-9._-]+", "-", text).strip("-")[:limit] or "run"


@dataclass(frozen=True)
class RunDir:
    dir: str

    @property
    def feed(self) -> str:
        return os.path.join(self.dir, "metrics.jsonl")

    @property
    def config(self) -> str:
        return os.path.join(self.dir, "config.yaml")

    @property
    def log(self) -> str:
        return os.path.join(self.dir, "train.log")

    @property
    def meta(self) -> str:
        return os.path.join(self.dir, "meta.json")

    @property
    def output(self) -> str:
        return os.path.join(self.dir, "output")

    @property
    def pid_file(self) -> str:
        return self.feed + ".pid"

    @property
    def id(self) -> str:
        return os.path.basename(self.dir)

    def write_meta(self, **meta: Any) -> Dict[str, Any]:
        meta.setdefault("started_at", time.time())
        with open(self.meta, "w") as f:
            json.dump(meta, f, indent=2, default=str)
        return meta

    def read_meta(self) -> Dict[str, Any]:
        try:
            with open(self.meta) as f:
                v = json.load(f)
            return v if isinstance(v, dict) else {}
        except (OSError, ValueError):
            return {}

    @staticmethod
    def of_feed(feed: str) -> "RunDir":
        return RunDir(os.path.dirname(os.path.abspath(feed)))


def new_run(label: str, root: Optional[str] = None, now: Optional[float] = None) -> RunDir:
    """A fresh run directory ``<stamp>-<label>``; a second run in the same second gets a numeric suffix."""
    base = runs_root(root)
    stamp = time.strftime("%Y%m%d-%H%M%S", time.localtime(now if now is not None else time.time()))
    name = f"{stamp}-{slug(label)}"
    path, n = os.path.join(base, name), 1
    while os.path.exists(path):
        n += 1
        path = os.path.join(base, f"{name}-{n}")
    os.makedirs(path)
    return RunDir(path)


def list_checkpoints(output_dir: str) -> List[Dict[str, Any]]:
    """``checkpoint-<step>`` / ``step_<step>`` directories of an output directory, newest first."""
    out = []
    try:
        names = os.listdir(output_dir)
    except OSError:
        return out
    for sub in [""] + [n for n in names if n == "checkpoints"]:
        d = os.path.join(output_dir, sub)
        for n in (os.listdir(d) if os.path.isdir(d) else []):
            m = re.fullmatch(r"(?:checkpoint-|step_)(\d+)", n)
            if m and os.path.isdir(os.path.join(d, n)):
                out.append({"name": os.path.join(sub, n) if sub else n, "step": int(m.group(1))})
    return sorted(out, key=lambda c: -c["step"])


def path_size(path: str) -> int:
    """Bytes below ``path``; symbolic links are not followed, so a cycle cannot recurse."""
    try:
        st = os.lstat(path)
    except OSError:
        return 0
    import stat

    if stat.S_ISLNK(st.st_mode):
        return 0
    if stat.S_ISREG(st.st_mode):
        return st.st_size
    if not stat.S_ISDIR(st.st_mode):
        return 0
    return sum(path_size(os.path.join(path, n)) for n in os.listdir(path))


def tail_bytes(path: str, limit: int = 16384) -> str:
    try:
        with open(path, "rb") as f:
            f.seek(0, os.SEEK_END)
            size = f.tell()
            f.seek(max(0, size - limit))
            return f.read().decode("utf-8", "replace")
    except OSError:
        return ""


def pid_alive(pid_file: str) -> bool:
    """True when the process recorded in ``pid_file`` still exists AND is the same process (same kernel start time), so a
    recycled pid of an unrelated program never counts as this run."""
    try:
        with open(pid_file) as f:
            rec = json.load(f)
        pid = int(rec["pid"])
        os.kill(pid, 0)
    except (OSError, ValueError, KeyError, TypeError):
        return False
    start = process_start_time(pid)
    return rec.get("start") is None or start is None or start == rec["start"]


def process_start_time(pid: int) -> Optional[int]:
    try:
        with open(f"/proc/{pid}/stat") as f:
            return int(f.read().rsplit(")", 1)[1].split()[19])
    except (OSError, ValueError, IndexError):
        return None


def write_pid_file(run: RunDir, pid: int) -> None:
    with open(run.pid_file, "w") as f:
        json.dump({"pid": pid, "start": process_start_time(pid)}, f)


def summarise_feed(feed: str) -> Dict[str, Any]:
    """Last step, last train / eval loss, best eval loss and record count of a feed file."""
    out: Dict[str, Any] = {"records": 0, "step": 0, "loss": None, "eval_loss": None, "best_eval_loss": None, "tokens_per_second": None}
    try:
        with open(feed) as f:
            for line in f:
                rec = parse_feed_line(line)
                if rec is None:
                    continue
                out["records"] += 1
                if "type" in rec:
                    continue
                out["step"] = max(out["step"], int(rec["step"]))
                if isinstance(rec.get("train/loss"), (int, float)):
                    out["loss"] = rec["train/loss"]
                if isinstance(rec.get("train/tokens_per_second"), (int, float)):
                    out["tokens_per_second"] = rec["train/tokens_per_second"]
                if isinstance(rec.get("eval/loss"), (int, float)):
                    out["eval_loss"] = rec["eval/loss"]
                    out["best_eval_loss"] = rec["eval/loss"] if out["best_eval_loss"] is None else min(out["best_eval_loss"], rec["eval/loss"])
    except OSError:
        pass
    return out


def list_runs(root: Optional[str] = None, now: Optional[float] = None, active_within_s: float = 60.0) -> List[Dict[str, Any]]:
    """The run history, newest first.  status: ``running`` (feed or log written recently, or the recorded local process is
    alive), ``done`` (reached ``max_steps``), ``stopped`` (has records, went quiet before the end), ``idle`` (no records)."""
    base, now = runs_root(root), now if now is not None else time.time()
    rows = []
    try:
        names = sorted(os.listdir(base), reverse=True)
    except OSError:
        return rows
    for n in names:
        run = RunDir(os.path.join(base, n))
        if not os.path.isdir(run.dir):
            continue
        meta, s = run.read_meta(), summarise_feed(run.feed)
        mtimes = [os.path.getmtime(p) for p in (run.feed, run.log) if os.path.exists(p)]
        age = now - max(mtimes) if mtimes else float("inf")
        max_steps = meta.get("max_steps")
        if pid_alive(run.pid_file) or age < active_within_s:
            status = "running"
        elif max_steps and s["step"] >= int(max_steps):
            status = "done"
        elif s["records"]:
            status = "stopped"
        else:
            status = "idle"
        remote = meta.get("remote") or {}
        rows.append({"run": n, "status": status, "mode": meta.get("mode", ""), "where": remote.get("kind", "local"), "model": meta.get("model", ""),
                     "step": s["step"], "max_steps": max_steps, "loss": s["loss"], "eval_loss": s["best_eval_loss"],
                     "checkpoints": len(list_checkpoints(run.output)), "dir": run.dir})
    return rows

"""``surogate monitor``: a live terminal dashboard over the JSON-lines metrics feed (``report_to: [surogate]``).

It does not import the training code: it tails the feed file (default ``/tmp/surogate_metrics.jsonl``), keeps a small state
(loss / learning-rate / throughput / gradient-norm series, evaluation points, the last GPU and MoE records) and redraws a
layout of panels: loss curve, step progress, throughput, GPUs (from the feed, or read live through NVML), MoE balance.
``--once`` renders a single frame (used by tests and for piping into a file); ``launch`` starts a run with the ``surogate``
command, locally or over SSH, and then monitors it; ``--interactive`` opens the paged dashboard (``cli/dashboard.py``).

Parity: jackalope/ (terminal dashboard that tails the same feed; its launch back ends are ``surogate_b200/launch`` behind ``surogate launch``).
"""
from __future__ import annotations

import argparse
import json
import os
import shlex
import subprocess
import sys
import time
from typing import Any, Dict, List, Optional

DEFAULT_FEED = "/tmp/surogate_metrics.jsonl"
BLOCKS = " ▁▂▃▄▅▆▇█"


class FeedState:
    """Incremental reader of the feed: ``poll()`` consumes the lines appended since the last call."""

    def __init__(self, path: str, keep: int = 4096):
        self.path, self.keep = path, keep
        self.offset = 0
        self.inode: Optional[int] = None
        self.steps: List[int] = []
        self.series: Dict[str, List[float]] = {"loss": [], "lr": [], "tps": [], "norm": []}
        self.evals: List[tuple] = []
        self.gpu: Dict[str, Any] = {}
        self.moe: Dict[str, Any] = {}
        self.max_steps: Optional[int] = None
        self.run_name = ""
        self.last_update = 0.0

    def poll(self) -> int:
        try:
            st = os.stat(self.path)
        except OSError:
            return 0
        if self.inode != st.st_ino or st.st_size < self.offset:  # a new run replaced or truncated the feed
            self.__init__(self.path, self.keep)
            self.inode = st.st_ino
        n = 0
        with open(self.path) as f:
            f.seek(self.offset)
            while True:
                line = f.readline()
                if not line or not line.endswith("\n"):
                    break  # a partially written last line is read on the next poll
                self.offset = f.tell()
                try:
                    self.consume(json.loads(line))
                    n += 1
                except (ValueError, TypeError):
                    continue
        if n:
            self.last_update = time.time()
        return n

    @staticmethod
    def normalise(rec: Dict[str, Any]) -> Dict[str, Any]:
        """A feed record in the dashboard schema (``train/loss``, ``type: gpu`` ...) as the ``{"log": kind, ...}`` form
        ``consume`` reads; records already in that form pass through."""
        if "log" in rec:
            return rec
        kind = rec.get("type")
        if kind == "config":
            return {"log": "options", "config": {k: v for k, v in rec.items() if k not in ("type", "ts")}}
        if kind in ("gpu", "moe"):
            out = {"log": kind, **{k: v for k, v in rec.items() if k != "type"}}
            if kind == "gpu":
                for ours, theirs in (("gpu_util", "gpu_utilization"), ("power_w", "power"), ("temperature_c", "temperature"), ("index", "gpu_id")):
                    if ours not in out and theirs in out:
                        out[ours] = out[theirs]
            return out
        if kind is None and "step" in rec:
            if any(k.startswith("eval/") for k in rec):
                return {"log": "eval", "step": rec["step"], "loss": rec.get("eval/loss", float("nan"))}
            return {"log": "step", "step": rec["step"], "loss": rec.get("train/loss"), "lr": rec.get("train/lr"),
                    "norm": rec.get("train/norm", rec.get("train/grad_norm")), "tps": rec.get("train/tokens_per_second"),
                    "max_steps": rec.get("max_steps"), "phase": rec.get("train/phase", rec.get("phase"))}
        return rec

    def consume(self, rec: Dict[str, Any]) -> None:
        rec = self.normalise(rec)
        kind = rec.get("log")
        if kind == "step":
            self.steps.append(int(rec.get("step", len(self.steps) + 1)))
            for k, src in (("loss", "loss"), ("lr", "lr"), ("tps", "tps"), ("norm", "norm")):
                v = rec.get(src)
                self.series[k].append(float(v) if isinstance(v, (int, float)) else float("nan"))
            if rec.get("max_steps"):
                self.max_steps = int(rec["max_steps"])
            if len(self.steps) > self.keep:
                self.steps = self.steps[-self.keep:]
                for k in self.series:
                    self.series[k] = self.series[k][-self.keep:]
        elif kind == "eval":
            self.evals.append((int(rec.get("step", 0)), float(rec.get("loss", float("nan")))))
        elif kind == "gpu":
            self.gpu = rec
        elif kind == "moe":
            self.moe = rec
        elif kind == "options":
            cfg = rec.get("config") or {}
            self.run_name = cfg.get("run_name") or self.run_name
            self.max_steps = cfg.get("max_steps") or self.max_steps


def chart(values: List[float], width: int, height: int) -> List[str]:
    """Block-character line chart of the last ``width`` buckets (bucket mean), ``height`` rows, with a y-axis label column."""
    vals = [v for v in values if v == v]
    if not vals:
        return ["(waiting for data)"]
    per = max(1, -(-len(vals) // width))
    buckets = [sum(vals[i:i + per]) / len(vals[i:i + per]) for i in range(0, len(vals), per)][-width:]
    lo, hi = min(buckets), max(buckets)
    span = (hi - lo) or 1.0
    rows = []
    for r in range(height):
        top, bot = hi - span * r / height, hi - span * (r + 1) / height
        cells = []
        for b in buckets:
            frac = (b - bot) / (top - bot) if top > bot else 0.0
            cells.append(BLOCKS[8] if frac >= 1 else BLOCKS[max(0, min(8, int(frac * 8)))] if frac > 0 else " ")
        label = f"{top:9.4g} ┤" if r in (0, height - 1) or r == height // 2 else " " * 9 + " │"
        rows.append(label + "".join(cells))
    return rows


def bar(frac: float, width: int = 16) -> str:
    frac = max(0.0, min(1.0, frac))
    full = int(frac * width)
    return "█" * full + "░" * (width - full)


def live_gpus() -> List[Dict[str, Any]]:
    try:
        from ..ops import host, host_available

        if host_available():
            out = []
            for i in range(16):
                g = host().query_gpu(i)
                if not g.get("ok"):
                    break
                out.append(dict(g, index=i))
            return out
    except Exception:  # noqa: BLE001 - no NVML on this machine: the GPU panel shows the feed's record only
        pass
    return []


def render(state: FeedState, width: int = 100, gpus: Optional[List[Dict[str, Any]]] = None) -> str:
    w = max(40, width)
    out = [f"◆ surogate monitor  {state.run_name}".ljust(w - 12) + ("● live" if time.time() - state.last_update < 30 else "○ idle")]
    out.append("─" * w)
    out.append("TRAINING LOSS")
    out += chart(state.series["loss"], w - 12, 8)
    if state.steps:
        step, total = state.steps[-1], state.max_steps
        prog = f"step {step}" + (f"/{total}  {bar(step / total, 24)} {100 * step / total:4.1f}%" if total else "")
        last = {k: (v[-1] if v else float("nan")) for k, v in state.series.items()}
        out.append(f"{prog}   loss {last['loss']:.4f}   lr {last['lr']:.3g}   grad-norm {last['norm']:.3g}   {last['tps'] / 1e3:.1f}k tok/s")
        tps = [v for v in state.series["tps"] if v == v]
        if tps:
            out.append("THROUGHPUT " + "".join(BLOCKS[max(1, min(8, int(8 * v / max(tps))))] for v in tps[-(w - 12):]))
    if state.evals:
        out.append("EVAL  " + "  ".join(f"{s}: {l:.4f}" for s, l in state.evals[-6:]))
    rows = gpus if gpus else ([state.gpu] if state.gpu else [])
    for i, g in enumerate(rows):
        util = float(g.get("gpu_util", g.get("util", 0)) or 0) / 100.0
        mem_used, mem_total = float(g.get("mem_used", g.get("memory_used", 0)) or 0), float(g.get("mem_total", g.get("memory_total", 0)) or 0)
        mem = f"  mem {mem_used / 2**30:.0f}/{mem_total / 2**30:.0f} GiB" if mem_total else ""
        out.append(f"gpu{g.get('index', i)} {bar(util)} {100 * util:3.0f}%{mem}  {g.get('power_w', g.get('power', ''))} W  {g.get('temperature_c', g.get('temperature', ''))} C")
    if state.moe:
        m = state.moe
        out.append(f"MoE  imbalance {m.get('imbalance', m.get('load_imbalance', float('nan'))):.2f}  aux {m.get('aux_loss', float('nan')):.4g}  "
                   f"dead experts {m.get('dead_experts', 0)}")
    return "\n".join(line[:w] for line in out)


def launch(config: str, command: str = "sft", ssh: Optional[str] = None, gpus: int = 0, extra: Optional[List[str]] = None) -> subprocess.Popen:
    """Start ``surogate <command> <config>`` in the background, locally or on ``ssh`` (user@host)."""
    base = [sys.executable, "-m", "surogate_b200.cli.main", command, config] + list(extra or [])
    if gpus > 1:
        base = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1", "-m",
                "surogate_b200.cli.main", command, config] + list(extra or [])
    if ssh:
        remote = " ".join(shlex.quote(a) for a in ["python"] + base[1:])
        base = ["ssh", ssh, remote]
    return subprocess.Popen(base, stdout=subprocess.DEVNULL, stderr=subprocess.STDOUT, start_new_session=True)


def browse_models(query: str, limit: int = 20, search=None) -> List[Dict[str, Any]]:
    """Models the Launch view can line up: a local path (``/...``, ``~/...``, ``./...``) lists the model directories below it,
    anything else is a HuggingFace search.  Each row says whether this framework can train the architecture.
    ``search(query, limit) -> [{"id", "architectures", "downloads"}]`` replaces the hub call (tests, air-gapped machines)."""
    from ..models.registry import describe_config, supported_architectures

    rows: List[Dict[str, Any]] = []
    if query.startswith(("/", "~", ".")):
        root = os.path.abspath(os.path.expanduser(query))
        cands = [root] + sorted(os.path.join(root, d) for d in os.listdir(root) if os.path.isdir(os.path.join(root, d))) if os.path.isdir(root) else []
        for d in cands:
            cfg_path = os.path.join(d, "config.json")
            if not os.path.exists(cfg_path):
                continue
            with open(cfg_path) as f:
                info = describe_config(json.load(f))
            rows.append({"id": d, "architecture": info["architecture"], "trainable": bool(info["supported"]), "moe": info["is_moe"],
                         "quant": (info["quant_info"] or {}).get("kind"), "layers": info["num_hidden_layers"], "hidden": info["hidden_size"]})
        return rows[:limit]
    if search is None:
        def search(q, n):
            from huggingface_hub import HfApi

            return [{"id": m.id, "architectures": ((getattr(m, "config", None) or {}).get("architectures") or []), "downloads": getattr(m, "downloads", 0)}
                    for m in HfApi().list_models(search=q, limit=n, sort="downloads", direction=-1, expand=["config", "downloads"])]
    ok = set(supported_architectures())
    for m in search(query, limit):
        arch = (m.get("architectures") or [""])[0]
        rows.append({"id": m["id"], "architecture": arch, "trainable": arch in ok, "downloads": m.get("downloads", 0)})
    return rows


def browse_datasets(query: str, limit: int = 20, search=None) -> List[Dict[str, Any]]:
    """Datasets for the Launch view: local ``.jsonl`` / ``.json`` / ``.parquet`` files below a path with the detected sample type,
    or a HuggingFace dataset search."""
    rows: List[Dict[str, Any]] = []
    if query.startswith(("/", "~", ".")):
        from ..data.datasets import detect_type

        root = os.path.abspath(os.path.expanduser(query))
        files = [root] if os.path.isfile(root) else sorted(os.path.join(root, f) for f in os.listdir(root)) if os.path.isdir(root) else []
        for f in files:
            if not f.endswith((".jsonl", ".json", ".parquet")):
                continue
            kind = None
            if f.endswith(".jsonl"):
                with open(f) as fh:
                    line = fh.readline().strip()
                try:
                    kind = detect_type(json.loads(line).keys()) if line else None
                except Exception:  # noqa: BLE001
                    kind = None
            rows.append({"id": f, "type": kind, "bytes": os.path.getsize(f)})
        return rows[:limit]
    if search is None:
        def search(q, n):
            from huggingface_hub import HfApi

            return [{"id": d.id, "downloads": getattr(d, "downloads", 0)} for d in HfApi().list_datasets(search=q, limit=n, sort="downloads", direction=-1)]
    return [{"id": d["id"], "downloads": d.get("downloads", 0)} for d in search(query, limit)]


def past_runs(root: str) -> List[Dict[str, Any]]:
    """Runs below ``root`` (output directories): last logged step and loss, checkpoints and exported model present."""
    rows = []
    for d in sorted(os.listdir(root)) if os.path.isdir(root) else []:
        path = os.path.join(root, d)
        if not os.path.isdir(path):
            continue
        logs = [f for f in os.listdir(path) if f.endswith(".jsonl")]
        ckpts = sorted(c for c in os.listdir(path) if c.startswith(("step_", "checkpoint")))
        last: Dict[str, Any] = {}
        for lf in logs:
            st = FeedState(os.path.join(path, lf))
            st.poll()
            if st.steps:
                last = {"step": st.steps[-1], "loss": st.series["loss"][-1]}
        if logs or ckpts or os.path.exists(os.path.join(path, "model.safetensors")) or os.path.exists(os.path.join(path, "config.json")):
            rows.append({"run": d, **last, "checkpoints": len(ckpts), "exported": os.path.exists(os.path.join(path, "config.json"))})
    return rows


def table(rows: List[Dict[str, Any]]) -> str:
    if not rows:
        return "(nothing found)"
    cols = list(dict.fromkeys(k for r in rows for k in r))
    cell = lambda v: ("yes" if v else "no") if isinstance(v, bool) else ("" if v is None else (f"{v:.4g}" if isinstance(v, float) else str(v)))  # noqa: E731
    w = {c: max(len(c), *(len(cell(r.get(c))) for r in rows)) for c in cols}
    lines = ["  ".join(c.ljust(w[c]) for c in cols), "  ".join("-" * w[c] for c in cols)]
    lines += ["  ".join(cell(r.get(c)).ljust(w[c]) for c in cols) for r in rows]
    return "\n".join(lines)


def main(argv, command: str = "monitor") -> int:
    p = argparse.ArgumentParser(prog="surogate monitor")
    p.add_argument("action", nargs="?", default="watch", choices=["watch", "launch", "models", "datasets", "runs"])
    p.add_argument("config", nargs="?", help="training config (launch) | search text or path (models, datasets) | output root (runs)")
    p.add_argument("--feed", default=DEFAULT_FEED)
    p.add_argument("--once", action="store_true", help="render one frame and exit")
    p.add_argument("--interval", type=float, default=1.0)
    p.add_argument("--ssh", default=None)
    p.add_argument("--gpus", type=int, default=0)
    p.add_argument("--command", default="sft")
    p.add_argument("--interactive", "-i", action="store_true", help="the paged dashboard (Monitor, GPUs, Models, Datasets, Launch, Runs) with keyboard navigation")
    p.add_argument("--runs-dir", default=None)
    a = p.parse_args(argv)
    if (a.interactive or (command == "jackalope" and a.action == "watch" and not a.once)) and sys.stdin.isatty():
        from .dashboard import Dashboard, run

        return run(Dashboard(a.feed, a.runs_dir))
    if a.action in ("models", "datasets", "runs"):
        if not a.config:
            p.error(f"{a.action} needs a search text or a path")
        print(table({"models": browse_models, "datasets": browse_datasets, "runs": past_runs}[a.action](a.config)))
        return 0
    if a.action == "launch":
        if not a.config:
            p.error("launch needs a config file")
        proc = launch(a.config, a.command, a.ssh, a.gpus)
        print(f"started pid {proc.pid}", file=sys.stderr)
    state = FeedState(a.feed)
    if a.once:
        state.poll()
        import shutil

        print(render(state, width=shutil.get_terminal_size((100, 30)).columns))
        return 0
    from rich.console import Console
    from rich.live import Live
    from rich.text import Text

    console = Console()
    with Live(Text(render(state, console.width)), console=console, refresh_per_second=4, screen=False) as live:
        try:
            while True:
                state.poll()
                live.update(Text(render(state, console.width, live_gpus())))
                time.sleep(a.interval)
        except KeyboardInterrupt:
            return 0

"""Loss / learning-rate / throughput plots from a run's JSON-lines log (PNG with matplotlib, text sparkline without).

Parity: surogate/train/training_plot.py.
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional

BARS = "▁▂▃▄▅▆▇█"


def read_log(path: str) -> Dict[str, List[dict]]:
    out: Dict[str, List[dict]] = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            try:
                r = json.loads(line)
            except json.JSONDecodeError:
                continue
            out.setdefault(r.get("log", "?"), []).append(r)
    return out


def sparkline(values: List[float], width: int = 60) -> str:
    if not values:
        return ""
    if len(values) > width:
        k = len(values) / width
        values = [sum(values[int(i * k):max(int(i * k) + 1, int((i + 1) * k))]) / max(1, len(values[int(i * k):max(int(i * k) + 1, int((i + 1) * k))])) for i in range(width)]
    lo, hi = min(values), max(values)
    span = (hi - lo) or 1.0
    return "".join(BARS[min(len(BARS) - 1, int((v - lo) / span * (len(BARS) - 1)))] for v in values)


def plot_run(log_path: str, out_png: Optional[str] = None) -> str:
    recs = read_log(log_path)
    steps = recs.get("step", [])
    loss = [r["loss"] for r in steps]
    summary = f"loss {sparkline(loss)}  ({loss[0]:.3f} -> {loss[-1]:.3f})" if loss else "no step records"
    if out_png and steps:
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
        except ImportError:
            return summary + "\n(matplotlib is not installed: no PNG written)"
        fig, ax = plt.subplots(3, 1, figsize=(9, 9), sharex=True)
        x = [r["step"] for r in steps]
        ax[0].plot(x, loss, label="train")
        ev = recs.get("eval", [])
        if ev:
            ax[0].plot([r["step"] for r in ev], [r["loss"] for r in ev], "o-", label="eval")
        ax[0].set_ylabel("loss")
        ax[0].legend()
        ax[1].plot(x, [r.get("lr", 0) for r in steps])
        ax[1].set_ylabel("learning rate")
        ax[2].plot(x, [r.get("tps", 0) for r in steps])
        ax[2].set_ylabel("tokens / s")
        ax[2].set_xlabel("step")
        fig.tight_layout()
        fig.savefig(out_png, dpi=120)
        plt.close(fig)
    return summary

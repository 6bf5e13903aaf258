"""Time per op kind over a run: ``SUROGATE_OP_PROFILE=1`` makes the executor time every op it dispatches (forward and backward
graphs; the block stack's ops are timed inside it), and the totals are printed to stderr when the process ends, or read with
``Executor.op_profile.rows()``.

Every timed op is bracketed by two events and a synchronisation, so launches no longer overlap with host work: the shares are the
signal, the step time under the profile is not.  CUDA-graph replay is switched off while the profile is on.

Parity: csrc/src/runtime/executor/compiled_ops_execute_backward.cpp:495 (report_backward_op_profile), :1020-1030, :1442, :1605-1612.
"""
from __future__ import annotations

import atexit
import os
import sys
import time
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch


class OpProfile:
    def __init__(self, device: torch.device, report_at_exit: bool = False):
        self.cuda = device.type == "cuda"
        self.total_ms: Dict[str, float] = {}
        self.count: Dict[str, int] = {}
        if self.cuda:
            self._start, self._end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if report_at_exit:
            atexit.register(self.report)

    def timed(self, kind: str, fn: Callable[..., Any], *args) -> Any:
        if self.cuda:
            self._start.record()
            out = fn(*args)
            self._end.record()
            self._end.synchronize()
            ms = self._start.elapsed_time(self._end)
        else:
            t0 = time.perf_counter()
            out = fn(*args)
            ms = (time.perf_counter() - t0) * 1e3
        self.total_ms[kind] = self.total_ms.get(kind, 0.0) + ms
        self.count[kind] = self.count.get(kind, 0) + 1
        return out

    def rows(self) -> List[Tuple[str, float, int, float, float]]:
        """(kind, total ms, calls, ms per call, share of the total), largest first."""
        whole = sum(self.total_ms.values()) or 1.0
        return sorted(((k, v, self.count[k], v / self.count[k], v / whole) for k, v in self.total_ms.items()), key=lambda r: -r[1])

    def reset(self) -> None:
        self.total_ms.clear()
        self.count.clear()

    def report(self, file=None, top: int = 40) -> None:
        rows = self.rows()
        if not rows:
            return
        file = file or sys.stderr
        print(f"[op-profile] {sum(r[1] for r in rows):.1f} ms in {sum(r[2] for r in rows)} timed ops", file=file)
        print(f"  {'op':<34}{'total ms':>12}{'calls':>9}{'ms/call':>11}{'share':>8}", file=file)
        for kind, total, n, per, share in rows[:top]:
            print(f"  {kind:<34}{total:>12.2f}{n:>9}{per:>11.4f}{share:>7.1%}", file=file)


def env_op_profile(device: torch.device) -> Optional[OpProfile]:
    v = os.environ.get("SUROGATE_OP_PROFILE")
    return OpProfile(device, report_at_exit=True) if v and v != "0" else None

"""Filesystem transport: one ``step_<n>.npz`` per training step, written atomically (temp file + rename).

Every trainer rank reads the same file and takes its slice of the rows, so no rank-to-rank traffic is needed; the
orchestrator deletes files older than the trainer's acknowledged step.

Parity: surogate/grpo/transport/filesystem.py.
"""
from __future__ import annotations

import json
import os
import time
from typing import Dict, Optional

import numpy as np


class FilesystemTransport:
    def __init__(self, directory: str):
        self.dir = directory
        os.makedirs(directory, exist_ok=True)

    def _path(self, step: int) -> str:
        return os.path.join(self.dir, f"step_{step:08d}.npz")

    def send(self, step: int, arrays: Dict[str, np.ndarray], meta: Optional[Dict] = None) -> str:
        tmp = self._path(step) + ".tmp"
        with open(tmp, "wb") as f:
            np.savez(f, __meta__=np.frombuffer(json.dumps(meta or {}).encode(), dtype=np.uint8), **arrays)
        os.replace(tmp, self._path(step))
        return self._path(step)

    def ready(self, step: int) -> bool:
        return os.path.exists(self._path(step))

    def receive(self, step: int, timeout_s: float = 3600.0, poll_s: float = 0.05):
        t0 = time.time()
        while not self.ready(step):
            if time.time() - t0 > timeout_s:
                raise TimeoutError(f"no rollout batch for step {step} within {timeout_s}s in {self.dir}")
            time.sleep(poll_s)
        with np.load(self._path(step)) as z:
            meta = json.loads(bytes(z["__meta__"]).decode()) if "__meta__" in z else {}
            return {k: z[k] for k in z.files if k != "__meta__"}, meta

    def ack(self, step: int) -> None:
        """Trainer side: everything up to ``step`` has been consumed."""
        with open(os.path.join(self.dir, "ack.tmp"), "w") as f:
            f.write(str(step))
        os.replace(os.path.join(self.dir, "ack.tmp"), os.path.join(self.dir, "ack"))

    def acked(self) -> int:
        try:
            with open(os.path.join(self.dir, "ack")) as f:
                return int(f.read().strip() or -1)
        except (FileNotFoundError, ValueError):
            return -1

    def cleanup(self, keep_from: int) -> None:
        for fn in os.listdir(self.dir):
            if fn.startswith("step_") and fn.endswith(".npz") and int(fn[5:13]) < keep_from:
                os.remove(os.path.join(self.dir, fn))

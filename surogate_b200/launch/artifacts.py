"""Bring a finished run's outputs (trained model, checkpoints, log) back under ``<run>/output``, by where the run ran:

  local   already in the run directory
  ssh     ``scp -r`` of the remote output directory
  modal   ``modal volume get`` of the run's Volume
  dstack  not possible (the instance is torn down): push to a hub from the config, or use SSH / Modal

Parity: jackalope/src/artifacts.ts.
"""
from __future__ import annotations

import os
import subprocess
from typing import Any, Callable, Dict, Optional

from .runs import RunDir
from .ssh import parse_target, scp_args


def fetchable(run: RunDir) -> bool:
    return (run.read_meta().get("remote") or {}).get("kind") in (None, "ssh", "modal")


def fetch_artifacts(run: RunDir, on_line: Optional[Callable[[str], None]] = None, runner=subprocess.run) -> Dict[str, Any]:
    remote = run.read_meta().get("remote")
    dest = run.output
    os.makedirs(dest, exist_ok=True)
    say = on_line or (lambda _l: None)

    def call(argv) -> bool:
        try:
            r = runner(argv, capture_output=True, text=True)
        except OSError as e:
            say(f"error: {e}")
            return False
        for line in ((r.stdout or "") + (r.stderr or "")).splitlines():
            say(line)
        return r.returncode == 0

    if not remote:
        return {"ok": True, "dest": dest}
    if remote.get("kind") == "ssh":
        t = parse_target(remote["host"])
        say(f"scp {t.host}:{remote['dir']}/output -> {dest}")
        ok = call(["scp", "-r", *scp_args(t), f"{t.host}:{remote['dir']}/output/.", dest])
        return {"ok": True, "dest": dest} if ok else {"ok": False, "reason": "scp failed; see the fetch log"}
    if remote.get("kind") == "modal":
        say(f"modal volume get {remote['session']} -> {dest}")
        ok = call(["modal", "volume", "get", "--force", remote["session"], "/model", dest])
        call(["modal", "volume", "get", "--force", remote["session"], "/train.log", dest])
        return {"ok": True, "dest": dest} if ok else {"ok": False, "reason": "`modal volume get` failed; see the fetch log"}
    return {"ok": False, "reason": "dstack runs cannot be downloaded (the instance is torn down): configure a hub push, or use SSH / Modal"}

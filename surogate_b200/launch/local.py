"""Start a run on this machine: the process is detached (a session of its own), its output goes to the run's log, its feed to the
run's feed file (``SUROGATE_METRICS_PATH``), its pid and kernel start time to a sidecar so ``stop`` ends exactly that process.

Parity: jackalope/src/launch.ts (spawnTraining, writePidFile), jackalope/src/local.ts.
"""
from __future__ import annotations

import json
import os
import signal
import subprocess
import sys
from typing import Any, Dict, List, Optional, Sequence

from .configs import load_overlaid, monitoring_overlay
from .runs import RunDir, new_run, pid_alive, write_pid_file


def surogate_argv(mode: str, config_path: str, n_gpus: int = 1, surogate_bin: Optional[str] = None) -> List[str]:
    """argv of ``surogate <mode> <config>``; several GPUs run one process per GPU under the torch launcher."""
    if surogate_bin:
        return [surogate_bin, mode, config_path]
    if n_gpus > 1:
        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n_gpus}", "--master-addr", "127.0.0.1",
                "-m", "surogate_b200.cli.main", mode, config_path]
    return [sys.executable, "-m", "surogate_b200.cli.main", mode, config_path]


def launch_local(config_text: str, label: str, gpu_ids: Sequence[int] = (), mode: str = "sft", root: Optional[str] = None,
                 surogate_bin: Optional[str] = None, popen=subprocess.Popen, extra_env: Optional[Dict[str, str]] = None) -> Dict[str, Any]:
    run = new_run(f"local-{label}", root)
    n = max(1, len(gpu_ids))
    text = monitoring_overlay(config_text, n, run.feed)
    cfg = load_overlaid(text)
    if "output_dir" not in cfg or str(cfg["output_dir"]).startswith("./"):
        text = text.rstrip() + f"\noutput_dir: {json.dumps(run.output)}\n"  # relative outputs land inside the run's own directory
    with open(run.config, "w") as f:
        f.write(text)
    env = dict(os.environ, SUROGATE_METRICS_PATH=run.feed, **(extra_env or {}))
    if gpu_ids:
        env["CUDA_VISIBLE_DEVICES"] = ",".join(str(g) for g in gpu_ids)
    log = open(run.log, "ab")
    try:
        proc = popen(surogate_argv(mode, run.config, n, surogate_bin), stdout=log, stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL,
                     env=env, cwd=run.dir, start_new_session=True)
    except OSError as e:
        return {"ok": False, "reason": str(e), "run": run}
    finally:
        log.close()
    write_pid_file(run, proc.pid)
    run.write_meta(mode=mode, label=f"local-{label}", model=cfg.get("model"), recipe=cfg.get("recipe"), gpus=list(gpu_ids),
                   max_steps=cfg.get("max_steps"), dataset=((cfg.get("datasets") or [{}])[0] or {}).get("path"))
    return {"ok": True, "run": run, "feed": run.feed, "pid": proc.pid}


def stop_local(run: RunDir, sig: int = signal.SIGTERM) -> bool:
    """Signal the run's process group, only if the recorded pid is still that process."""
    if not pid_alive(run.pid_file):
        return False
    with open(run.pid_file) as f:
        pid = int(json.load(f)["pid"])
    try:
        os.killpg(os.getpgid(pid), sig)
    except OSError:
        return False
    return True

"""Run on a remote GPU server over SSH: the config is copied into a run directory on the host, the trainer starts inside a
detached ``tmux`` session (it survives the connection), and its feed and log are mirrored back with ``tail -F`` under a reconnect
loop.  Every ssh call is non-interactive with a short connect timeout and keep-alives, so a dead host fails fast instead of
hanging the caller.

Parity: jackalope/src/ssh.ts.
"""
from __future__ import annotations

import os
import re
import shlex
import subprocess
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from .configs import load_overlaid
from .runs import RunDir, new_run
from .stream import Mirror, register

GPU_QUERY = ["--query-gpu=index,name,memory.total,memory.used,utilization.gpu,compute_cap", "--format=csv,noheader,nounits"]


@dataclass
class SshTarget:
    host: str                      # user@host or an alias of the user's ssh config
    port: Optional[int] = None
    identity_file: Optional[str] = None
    workdir: str = "~/.surogate-watch/remote"


def parse_target(text: str) -> SshTarget:
    """``user@host:port`` / ``host`` / an alias."""
    t = text.strip()
    m = re.fullmatch(r"(.*?):(\d+)", t)
    return SshTarget(m.group(1), int(m.group(2))) if m else SshTarget(t)


def ssh_args(t: SshTarget) -> List[str]:
    a = ["-o", "BatchMode=yes", "-o", "ConnectTimeout=10", "-o", "ServerAliveInterval=15", "-o", "ServerAliveCountMax=3"]
    if t.port:
        a += ["-p", str(t.port)]
    if t.identity_file:
        a += ["-i", t.identity_file]
    return a


def scp_args(t: SshTarget) -> List[str]:
    a = ["-o", "BatchMode=yes", "-o", "ConnectTimeout=10"]
    if t.port:
        a += ["-P", str(t.port)]
    if t.identity_file:
        a += ["-i", t.identity_file]
    return a


def remote_launch_command(remote_dir: str, session: str, mode: str = "sft", surogate_bin: str = "surogate", gpu_ids=()) -> str:
    """The shell line run on the host: a detached tmux session that runs the trainer with its feed inside the run directory."""
    gpus = f"CUDA_VISIBLE_DEVICES={','.join(str(g) for g in gpu_ids)} " if gpu_ids else ""
    inner = f"cd {remote_dir} && {gpus}SUROGATE_METRICS_PATH={remote_dir}/metrics.jsonl {surogate_bin} {mode} config.yaml > train.log 2>&1 < /dev/null"
    return f"mkdir -p {remote_dir} && tmux new-session -d -s {session} {shlex.quote(inner)}"


def parse_gpu_csv(text: str) -> List[Dict[str, Any]]:
    rows = []
    for line in text.splitlines():
        cells = [c.strip() for c in line.split(",")]
        if len(cells) < 2 or not cells[0].isdigit():
            continue

        def num(i):
            try:
                return float(cells[i])
            except (IndexError, ValueError):
                return None

        rows.append({"index": int(cells[0]), "name": cells[1], "mem_mb": num(2), "mem_used_mb": num(3), "util": num(4), "compute_cap": num(5)})
    return rows


def detect_remote_gpus(t: SshTarget, run=subprocess.run) -> List[Dict[str, Any]]:
    r = run(["ssh", *ssh_args(t), t.host, "nvidia-smi", *GPU_QUERY], capture_output=True, text=True, timeout=15)
    if r.returncode != 0:
        raise RuntimeError((r.stderr or "ssh failed").strip().splitlines()[-1])
    return parse_gpu_csv(r.stdout)


def follow_command(t: SshTarget, remote_path: str):
    """argv factory for ``Mirror``: print the remote file from a byte offset on, then follow it."""
    return lambda offset: ["ssh", *ssh_args(t), t.host, "tail", "-c", f"+{offset + 1}", "-F", remote_path]


def launch_remote(t: SshTarget, config_text: str, label: str, mode: str = "sft", surogate_bin: str = "surogate", gpu_ids=(),
                  root: Optional[str] = None, run=subprocess.run, mirror: bool = True) -> Dict[str, Any]:
    rd = new_run(f"ssh-{label}", root)
    remote_dir = f"{t.workdir}/{rd.id}"
    session = re.sub(r"[^A-Za-z0-9_]", "_", f"sur_{rd.id}")
    with open(rd.config, "w") as f:
        f.write(config_text)
    steps = [
        (["ssh", *ssh_args(t), t.host, f"mkdir -p {remote_dir}"], 15),
        (["scp", *scp_args(t), rd.config, f"{t.host}:{remote_dir}/config.yaml"], 30),
        (["ssh", *ssh_args(t), t.host, remote_launch_command(remote_dir, session, mode, surogate_bin, gpu_ids)], 20),
    ]
    for argv, limit in steps:
        try:
            r = run(argv, capture_output=True, text=True, timeout=limit)
        except (OSError, subprocess.TimeoutExpired) as e:
            return {"ok": False, "reason": str(e).splitlines()[0], "run": rd}
        if r.returncode != 0:
            return {"ok": False, "reason": ((r.stderr or "").strip().splitlines() or [f"{argv[0]} failed"])[-1], "run": rd}
    cfg = load_overlaid(config_text)
    rd.write_meta(mode=mode, label=f"ssh-{label}", model=cfg.get("model"), recipe=cfg.get("recipe"), max_steps=cfg.get("max_steps"),
                  remote={"kind": "ssh", "host": t.host if not t.port else f"{t.host}:{t.port}", "session": session, "dir": remote_dir})
    mirrors = []
    if mirror:
        for remote, local in ((f"{remote_dir}/metrics.jsonl", rd.feed), (f"{remote_dir}/train.log", rd.log)):
            m = Mirror(follow_command(t, remote), local).start()
            register(m)
            mirrors.append(m)
    return {"ok": True, "run": rd, "feed": rd.feed, "session": session, "host": t.host, "mirrors": mirrors}


def stop_remote(t: SshTarget, session: str, popen=subprocess.Popen) -> bool:
    """End the run by killing its tmux session; fire and forget, so a slow host cannot block the caller."""
    if not re.fullmatch(r"[A-Za-z0-9_.-]+", session):
        return False
    try:
        popen(["ssh", *ssh_args(t), t.host, f"tmux kill-session -t {session}"], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL,
              stdin=subprocess.DEVNULL, start_new_session=True)
    except OSError:
        return False
    return True


def recent_hosts(path: Optional[str] = None, remember: Optional[str] = None, keep: int = 6) -> List[str]:
    """Recently used targets, newest first; ``remember`` puts a host at the front."""
    path = path or os.path.join(os.path.expanduser("~"), ".surogate-watch", "ssh-hosts")
    try:
        with open(path) as f:
            hosts = [l.strip() for l in f if l.strip()]
    except OSError:
        hosts = []
    if remember and remember.strip():
        h = remember.strip()
        hosts = ([h] + [x for x in hosts if x != h])[:keep]
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "w") as f:
            f.write("\n".join(hosts) + "\n")
    return hosts[:keep]

"""One-command GRPO: ``surogate grpo-train`` (rollout engine and trainer on disjoint GPU sets) and ``surogate grpo-colocate``
(both on the same GPUs, the engine's memory share capped so the trainer fits beside it).

Both runners start the three components of asynchronous GRPO as child processes of one supervisor:

    rollout engine  ``surogate grpo-infer``  CUDA_VISIBLE_DEVICES = inference GPUs (split) / all GPUs (colocate)
    trainer         ``surogate grpo``        CUDA_VISIBLE_DEVICES = trainer GPUs; torchrun when more than one
    orchestrator    ``surogate grpo-orch``   no GPU

Every child gets its own process group, so tearing one down takes its workers (tensor-parallel engine ranks, torchrun ranks)
with it.  The supervisor waits on all of them: the first child to exit with an error, or the trainer finishing, ends the run;
the rest get SIGTERM, a grace period, then SIGKILL, addressed by process-group id (never by name).  GPU sets are validated
before anything is spawned: disjoint in split mode, sized to the engine's tensor-parallel x data-parallel topology.

In colocate mode the trainer publishes weights through CUDA IPC handles (``weight_broadcast.ColocateBroadcast``) when the
engine runs in a process this supervisor created with a queue, else through the filesystem like split mode.  The reference
additionally lets the trainer *borrow* the engine's quantised base weights over IPC; here the trainer keeps its own (QLoRA)
base and only the adapters travel.

Parity: surogate/grpo/split.py:129-494 (grpo_split, GPU-set checks, tree teardown), surogate/grpo/colocate.py:1-479.
"""
from __future__ import annotations

import os
import signal
import subprocess
import sys
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple


def parse_gpu_ids(spec: Optional[str]) -> List[int]:
    if spec is None or str(spec).strip() == "":
        return []
    out: List[int] = []
    for part in str(spec).split(","):
        part = part.strip()
        if "-" in part:
            a, b = part.split("-", 1)
            out += list(range(int(a), int(b) + 1))
        elif part:
            out.append(int(part))
    if len(set(out)) != len(out):
        raise ValueError(f"GPU list '{spec}' names a device twice")
    return out


def check_disjoint(*labelled: Tuple[str, Sequence[int]]) -> None:
    seen: Dict[int, str] = {}
    for label, ids in labelled:
        for i in ids:
            if i in seen:
                raise ValueError(f"GPU {i} is assigned to both {seen[i]} and {label}; split mode needs disjoint sets (use grpo-colocate to share GPUs)")
            seen[i] = label


def check_topology(label: str, ids: Sequence[int], tensor_parallel: int, data_parallel: int = 1) -> None:
    need = tensor_parallel * data_parallel
    if len(ids) != need:
        raise ValueError(f"{label}: {len(ids)} GPUs given but tensor_parallel_size {tensor_parallel} x data_parallel_size {data_parallel} needs {need}")


@dataclass
class Component:
    name: str
    argv: List[str]
    env: Dict[str, str] = field(default_factory=dict)
    essential: bool = True          # its exit ends the run
    ends_run_on_success: bool = False   # the trainer: exit 0 means the job is done
    proc: Optional[subprocess.Popen] = None


PR_SET_CHILD_SUBREAPER = 36  # <linux/prctl.h>


def set_child_subreaper() -> bool:
    """Make this process the reaper of its orphaned descendants (``prctl(PR_SET_CHILD_SUBREAPER)``): a worker whose parent dies
    mid-run then re-parents to the supervisor instead of to PID 1, so it stays inside the tree that the final walk of ``stop_all``
    sees.  Engine workers started by ``multiprocessing`` spawn are the case in point: they sit outside the engine's session group
    and outlive a ``killpg``.  Best effort: False where the call does not exist.
    Parity: docs/superpowers/specs/2026-07-06-grpo-vllm-subprocess-reap-design.md (surogate/grpo/split.py)."""
    try:
        import ctypes

        libc = ctypes.CDLL("libc.so.6", use_errno=True)
        return libc.prctl(PR_SET_CHILD_SUBREAPER, 1, 0, 0, 0) == 0
    except (OSError, AttributeError):
        return False


def reap_descendants(grace_s: float = 5.0, log=print, exclude=()) -> int:
    """SIGTERM, then after ``grace_s`` SIGKILL, every process that is still a descendant of this one; by PID, so neither the
    launching shell (a parent, never a descendant) nor anybody else's process can be hit.  Returns how many were found."""
    try:
        import psutil
    except ImportError:
        return 0
    survivors = [p for p in psutil.Process().children(recursive=True) if p.pid not in exclude and p.is_running() and p.status() != psutil.STATUS_ZOMBIE]
    for p in survivors:
        try:
            p.terminate()
        except psutil.Error:
            pass
    _, alive = psutil.wait_procs(survivors, timeout=grace_s)
    for p in alive:
        try:
            log(f"[grpo] pid {p.pid} ({p.name()}) survived SIGTERM: SIGKILL")
            p.kill()
        except psutil.Error:
            pass
    psutil.wait_procs(alive, timeout=grace_s)
    return len(survivors)


class Supervisor:
    def __init__(self, components: Sequence[Component], grace_s: float = 10.0, poll_s: float = 0.2, log=print, reap: bool = False):
        """``reap``: own the whole descendant tree (subreaper flag at start, a final walk that ends every descendant that was not
        there before ``start``).  The command-line runs switch it on; a program that embeds a supervisor next to children of its
        own leaves it off."""
        self.components, self.grace, self.poll, self.log, self.reap = list(components), grace_s, poll_s, log, reap
        self._before: set = set()

    def start(self) -> None:
        if self.reap:
            set_child_subreaper()   # before the first child: orphans of the components come back to this process
            try:
                import psutil

                self._before = {p.pid for p in psutil.Process().children(recursive=True)}
            except ImportError:
                pass
        for c in self.components:
            env = dict(os.environ)
            env.update(c.env)
            c.proc = subprocess.Popen(c.argv, env=env, start_new_session=True)   # own session = own process group
            self.log(f"[grpo] started {c.name} (pid {c.proc.pid})" + (f" on GPUs {c.env['CUDA_VISIBLE_DEVICES']}" if "CUDA_VISIBLE_DEVICES" in c.env else ""))

    def _signal_group(self, c: Component, sig: int) -> None:
        if c.proc is None or c.proc.poll() is not None:
            return
        try:
            os.killpg(c.proc.pid, sig)      # pid == pgid: the child leads its own session
        except ProcessLookupError:
            pass

    def stop_all(self) -> None:
        for c in self.components:
            self._signal_group(c, signal.SIGTERM)
        deadline = time.time() + self.grace
        while time.time() < deadline and any(c.proc is not None and c.proc.poll() is None for c in self.components):
            time.sleep(self.poll)
        for c in self.components:
            if c.proc is not None and c.proc.poll() is None:
                self.log(f"[grpo] {c.name} ignored SIGTERM for {self.grace:.0f}s: SIGKILL to its process group")
                self._signal_group(c, signal.SIGKILL)
        for c in self.components:
            if c.proc is not None:
                try:
                    c.proc.wait(timeout=self.grace)
                except subprocess.TimeoutExpired:
                    pass
        if self.reap:   # workers that left their component's process group (re-parented to this process by the subreaper flag)
            n = reap_descendants(min(self.grace, 5.0), self.log, exclude=self._before)
            if n:
                self.log(f"[grpo] reaped {n} leftover process(es)")

    def wait(self, timeout_s: Optional[float] = None) -> int:
        """Returns the run's exit code: 0 when the trainer finished, else the failing component's code."""
        t0 = time.time()
        rc = 0
        try:
            while True:
                for c in self.components:
                    code = c.proc.poll() if c.proc is not None else None
                    if code is None:
                        continue
                    if code == 0 and c.ends_run_on_success:
                        self.log(f"[grpo] {c.name} finished")
                        return 0
                    if code != 0 and c.essential:
                        self.log(f"[grpo] {c.name} exited with code {code}: stopping the other components")
                        rc = code if code > 0 else 128 - code
                        return rc
                    if code == 0 and c.essential and not c.ends_run_on_success and c.name != "orchestrator":
                        self.log(f"[grpo] {c.name} exited although the run is not over: stopping")
                        return 1
                if timeout_s is not None and time.time() - t0 > timeout_s:
                    self.log("[grpo] supervisor timeout")
                    return 124
                time.sleep(self.poll)
        except KeyboardInterrupt:
            return 130
        finally:
            self.stop_all()

    def run(self, timeout_s: Optional[float] = None) -> int:
        self.start()
        return self.wait(timeout_s)


def _cli(command: str, config: str, extra: Sequence[str] = ()) -> List[str]:
    return [sys.executable, "-m", "surogate_b200.cli.main", command, config, *extra]


def _trainer_argv(config: str, n_gpus: int, master_port: int, extra: Sequence[str] = ()) -> List[str]:
    if n_gpus <= 1:
        return _cli("grpo", config, extra)
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n_gpus}", "--master-addr", "127.0.0.1", "--master-port", str(master_port),
            "-m", "surogate_b200.cli.main", "grpo", config, *extra]


def plan_split(train_cfg: str, infer_cfg: str, orch_cfg: str, trainer_gpus: str, vllm_gpus: str, tensor_parallel: int = 1, data_parallel: int = 1,
               judge_cfg: Optional[str] = None, judge_gpus: Optional[str] = None, judge_tensor_parallel: int = 1, master_port: int = 29631,
               max_steps: Optional[int] = None) -> List[Component]:
    tg, vg, jg = parse_gpu_ids(trainer_gpus), parse_gpu_ids(vllm_gpus), parse_gpu_ids(judge_gpus)
    if not tg or not vg:
        raise ValueError("grpo-train needs --trainer-gpus and --vllm-gpus")
    check_disjoint(("trainer", tg), ("rollout engine", vg), ("judge engine", jg))
    check_topology("rollout engine", vg, tensor_parallel, data_parallel)
    if (judge_cfg is None) != (not jg):
        raise ValueError("a judge engine needs both --judge-config and --judge-gpus")
    extra = ["--max-steps", str(max_steps)] if max_steps else []
    gl = lambda ids: ",".join(map(str, ids))  # noqa: E731
    comps = [Component("rollout engine", _cli("grpo-infer", infer_cfg), {"CUDA_VISIBLE_DEVICES": gl(vg)})]
    if judge_cfg is not None:
        check_topology("judge engine", jg, judge_tensor_parallel)
        comps.append(Component("judge engine", _cli("grpo-infer", judge_cfg), {"CUDA_VISIBLE_DEVICES": gl(jg)}))
    comps.append(Component("trainer", _trainer_argv(train_cfg, len(tg), master_port, extra), {"CUDA_VISIBLE_DEVICES": gl(tg)}, ends_run_on_success=True))
    comps.append(Component("orchestrator", _cli("grpo-orch", orch_cfg, extra), {"CUDA_VISIBLE_DEVICES": ""}))
    return comps


def plan_colocate(train_cfg: str, infer_cfg: str, orch_cfg: str, gpus: Optional[str] = None, master_port: int = 29632, max_steps: Optional[int] = None,
                  engine_memory_fraction: Optional[float] = None) -> List[Component]:
    ids = parse_gpu_ids(gpus)
    env = {"CUDA_VISIBLE_DEVICES": ",".join(map(str, ids))} if ids else {}
    extra = ["--max-steps", str(max_steps)] if max_steps else []
    infer_env = dict(env)
    if engine_memory_fraction is not None:
        if not 0.05 <= engine_memory_fraction <= 0.9:
            raise ValueError("engine_memory_fraction must leave room for the trainer: 0.05 .. 0.9")
        infer_env["SUROGATE_ENGINE_MEMORY_FRACTION"] = str(engine_memory_fraction)
    n = max(1, len(ids))
    return [Component("rollout engine", _cli("grpo-infer", infer_cfg), infer_env),
            Component("trainer", _trainer_argv(train_cfg, n, master_port, extra), dict(env, SUROGATE_GRPO_COLOCATE="1"), ends_run_on_success=True),
            Component("orchestrator", _cli("grpo-orch", orch_cfg, extra), {"CUDA_VISIBLE_DEVICES": ""})]

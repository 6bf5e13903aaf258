"""Failure detection for process-per-GPU jobs: heartbeats, root-cause propagation, abort instead of hang.

Every rank runs a small daemon thread that (a) writes a heartbeat (step, wall time) to the job's key-value store and
(b) watches the other ranks' heartbeats and failure notes.  A rank that raises inside ``guard()`` publishes its traceback
under ``fail/<rank>`` before it dies, so the survivors report *why* the job ended ("rank 3 failed: CUDA out of memory ...")
rather than a collective time-out.  A rank that disappears without a note (killed, wedged) is detected by a stale heartbeat.
On detection the watcher records the failure; the training loop sees it at its next ``check()`` — called before every
step's first collective — and raises ``RemoteRankFailed``; if the main thread is already stuck inside a collective the
process group's own time-out ends the wait, and ``abort_after`` seconds after detection the watcher force-exits the
process (exit code 134) so that a wedged job cannot linger on its GPUs.

Recovery is restart + resume: the launcher restarts the job and ``resume_from_checkpoint`` picks up the latest complete
checkpoint (``io/checkpoint.py: find_latest_checkpoint`` skips directories without ``checkpoint.json``).

Parity: csrc/src/utilities/comm.cpp:1477-1565 (first-failure tracking, abort on a detached thread), :1827-1836 (heartbeat),
csrc/src/binding/py_train.cpp:1919-1948 (lost-wakeup watchdog, force exit).
"""
from __future__ import annotations

import contextlib
import json
import os
import threading
import time
import traceback
from typing import Callable, Dict, Optional


class RemoteRankFailed(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} failed: {reason}")
        self.rank, self.reason = rank, reason


class DictStore:
    """In-process stand-in for a distributed key-value store (tests, single-process runs)."""

    def __init__(self):
        self.d: Dict[str, bytes] = {}
        self.lock = threading.Lock()

    def set(self, k: str, v) -> None:
        with self.lock:
            self.d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k: str) -> bytes:
        with self.lock:
            return self.d[k]

    def check(self, keys) -> bool:
        with self.lock:
            return all(k in self.d for k in keys)


def job_store(timeout_s: float = 30.0):
    """A TCPStore shared by all ranks of a torchrun job (rank 0 hosts it on MASTER_PORT + 1)."""
    import datetime

    import torch.distributed as dist

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    host, port = os.environ.get("MASTER_ADDR", "127.0.0.1"), int(os.environ.get("MASTER_PORT", "29500")) + 1
    return dist.TCPStore(host, port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=timeout_s), wait_for_workers=False)


class Watchdog:
    def __init__(self, store, rank: int, world: int, heartbeat_s: float = 1.0, stale_after_s: float = 45.0, abort_after_s: Optional[float] = 15.0,
                 on_abort: Optional[Callable[[str], None]] = None, prefix: str = "wd"):
        self.store, self.rank, self.world = store, rank, world
        self.heartbeat_s, self.stale_after_s, self.abort_after_s = heartbeat_s, stale_after_s, abort_after_s
        self.on_abort = on_abort or self._exit
        self.prefix = prefix
        self.step = 0
        self.failure: Optional[RemoteRankFailed] = None
        self.detected_at: Optional[float] = None
        self._stop = threading.Event()
        self._acknowledged = False
        self._thread: Optional[threading.Thread] = None
        self._seen: Dict[int, float] = {}

    # ------------------------------------------------------------------ keys
    def _k(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    @staticmethod
    def _exit(reason: str) -> None:  # pragma: no cover - ends the process
        print(f"[watchdog] aborting: {reason}", flush=True)
        os._exit(134)

    # ------------------------------------------------------------------ life cycle
    def start(self) -> "Watchdog":
        self._beat()
        self._thread = threading.Thread(target=self._run, name="surogate-watchdog", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        try:
            self.store.set(self._k("done", self.rank), b"1")
        except Exception:  # noqa: BLE001
            pass
        if self._thread is not None:
            self._thread.join(timeout=2 * self.heartbeat_s + 1)

    # ------------------------------------------------------------------ API for the training loop
    def tick(self, step: int) -> None:
        self.step = step

    def check(self) -> None:
        """Raise if another rank has failed or gone silent.  Call between steps, before the first collective."""
        if self.failure is not None:
            self._acknowledged = True
            raise self.failure

    def report_failure(self, exc: BaseException) -> None:
        note = {"type": type(exc).__name__, "message": str(exc)[:2000], "trace": traceback.format_exc()[-4000:], "step": self.step, "time": time.time()}
        try:
            self.store.set(self._k("fail", self.rank), json.dumps(note).encode())
        except Exception:  # noqa: BLE001
            pass

    @contextlib.contextmanager
    def guard(self):
        """Publish the root cause if the body raises (then re-raise)."""
        try:
            yield self
        except RemoteRankFailed:
            raise
        except BaseException as e:  # noqa: BLE001
            self.report_failure(e)
            raise

    # ------------------------------------------------------------------ watcher thread
    def _beat(self) -> None:
        try:
            self.store.set(self._k("hb", self.rank), json.dumps({"step": self.step, "time": time.time()}).encode())
        except Exception:  # noqa: BLE001
            pass

    def _peer_state(self, r: int):
        try:
            if self.store.check([self._k("fail", r)]):
                return "failed", json.loads(self.store.get(self._k("fail", r)).decode())
            if self.store.check([self._k("done", r)]):
                return "done", None
            if self.store.check([self._k("hb", r)]):
                return "alive", json.loads(self.store.get(self._k("hb", r)).decode())
        except Exception as e:  # noqa: BLE001  (store host gone = rank 0 gone)
            return "store_error", str(e)
        return "unknown", None

    def _run(self) -> None:
        started = time.time()
        while not self._stop.wait(self.heartbeat_s):
            self._beat()
            now = time.time()
            if self.failure is None:
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    state, info = self._peer_state(r)
                    if state == "failed":
                        self.failure = RemoteRankFailed(r, f"{info.get('type')}: {info.get('message')} (at step {info.get('step')})")
                    elif state == "alive":
                        last = self._seen.get(r)
                        if last is None or info["time"] > last:
                            self._seen[r] = info["time"]
                        if now - self._seen[r] > self.stale_after_s:
                            self.failure = RemoteRankFailed(r, f"no heartbeat for {now - self._seen[r]:.0f} s (last at step {info.get('step')})")
                    elif state == "unknown" and now - started > self.stale_after_s:
                        self.failure = RemoteRankFailed(r, "never sent a heartbeat")
                    elif state == "store_error" and r == 0 and now - started > self.stale_after_s:
                        self.failure = RemoteRankFailed(0, f"job store unreachable ({info})")
                    if self.failure is not None:
                        self.detected_at = now
                        break
            elif self.abort_after_s is not None and not self._acknowledged and now - self.detected_at > self.abort_after_s:
                self.on_abort(str(self.failure))  # the main thread is stuck (e.g. inside a collective): do not linger
                return


def install(rank: int, world: int, **kw) -> Optional[Watchdog]:
    """Watchdog over the job's TCP store for multi-rank runs (None for a single process)."""
    if world <= 1:
        return None
    return Watchdog(job_store(), rank, world, **kw).start()

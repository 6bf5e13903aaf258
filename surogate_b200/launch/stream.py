"""Plumbing shared by the streaming targets.

``pump_metrics`` reads a child's standard output on a thread: every line goes to the run log, lines that are feed records also go
to the run's feed file, so the monitor works on a cloud run unchanged.  ``Mirror`` keeps a local copy of a remote file current by
running a follow command (``ssh host tail -F``) and restarting it with back-off when the link drops, skipping the bytes it has
already written so a reconnect does not duplicate records.

Parity: jackalope/src/feed-pipe.ts, jackalope/src/ssh.ts (mirrorRemoteFile).
"""
from __future__ import annotations

import subprocess
import threading
from typing import Callable, List, Optional, Sequence

from .records import parse_feed_line


def pump_metrics(proc: subprocess.Popen, feed_path: str, log_path: str, on_line: Optional[Callable[[str], None]] = None) -> threading.Thread:
    """Start the pump for ``proc`` (created with ``stdout=PIPE, stderr=STDOUT`` or ``stderr=PIPE``); returns the stdout thread,
    which ends when the child closes its output."""

    def run_out():
        with open(feed_path, "a") as feed, open(log_path, "ab") as log:
            for raw in iter(proc.stdout.readline, b""):
                log.write(raw)
                log.flush()
                line = raw.decode("utf-8", "replace").rstrip("\r\n")
                if parse_feed_line(line) is not None:
                    feed.write(line + "\n")
                    feed.flush()
                elif on_line is not None:
                    on_line(line)

    def run_err():
        with open(log_path, "ab") as log:
            for raw in iter(proc.stderr.readline, b""):
                log.write(raw)
                log.flush()

    t = threading.Thread(target=run_out, name="feed-pump", daemon=True)
    t.start()
    if proc.stderr is not None and proc.stderr is not proc.stdout:
        threading.Thread(target=run_err, name="log-pump", daemon=True).start()
    return t


class Mirror:
    """Follow a remote file into ``local_path``.  ``command(offset)`` returns the argv that prints the remote file from byte
    ``offset`` on and keeps following it."""

    def __init__(self, command: Callable[[int], Sequence[str]], local_path: str, backoff: Sequence[float] = (1.0, 2.0, 5.0),
                 popen=subprocess.Popen):
        self.command, self.local_path, self.backoff = command, local_path, tuple(backoff)
        self._popen = popen
        self.stopped = threading.Event()
        self.attempts = 0
        self.bytes = 0
        self._proc: Optional[subprocess.Popen] = None
        self._thread: Optional[threading.Thread] = None

    def _loop(self) -> None:
        while not self.stopped.is_set():
            try:
                self._proc = self._popen(list(self.command(self.bytes)), stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, stdin=subprocess.DEVNULL)
            except OSError:
                self._proc = None
            if self._proc is not None:
                with open(self.local_path, "ab") as out:
                    while True:
                        chunk = self._proc.stdout.read1(65536) if hasattr(self._proc.stdout, "read1") else self._proc.stdout.read(65536)
                        if not chunk:
                            break
                        out.write(chunk)
                        out.flush()
                        self.bytes += len(chunk)
                self._proc.wait()
            if self.stopped.is_set():
                break
            delay = self.backoff[min(self.attempts, len(self.backoff) - 1)]
            self.attempts += 1
            self.stopped.wait(delay)

    def start(self) -> "Mirror":
        self._thread = threading.Thread(target=self._loop, name="mirror", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self.stopped.set()
        p = self._proc
        if p is not None and p.poll() is None:
            p.terminate()
        if self._thread is not None:
            self._thread.join(timeout=5)


_LIVE: List[object] = []  # pumps and mirrors of this process, ended by stop_all()


def register(handle) -> None:
    _LIVE.append(handle)


def stop_all() -> None:
    for h in _LIVE:
        stop = getattr(h, "stop", None) or getattr(h, "terminate", None)
        if stop is not None:
            try:
                stop()
            except OSError:
                pass
    _LIVE.clear()

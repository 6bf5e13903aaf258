"""Rollout scheduler: keeps a bounded number of generation requests in flight across inference servers, tracks which policy
version produced every rollout, and assembles trainer batches.

* ``max_inflight`` group requests are outstanding at any time; a finished group is replaced at once (continuous batching on the
  inference side stays full while the trainer works).
* Every request is pinned to the policy version current when it was issued.  When the trainer publishes a new version
  (``on_policy_update``), requests that would become more than ``max_off_policy_steps`` versions stale are cancelled and their
  prompts re-queued; the rest finish and are tagged with their off-policy level.
* ``max_async_level`` bounds how far generation may run ahead of the trainer: ``may_issue(step)`` is false while
  ``step - trainer_version > max_async_level``.
* A batch is complete when ``batch_size`` rollouts (or ``token_batch_size`` tokens) are ready; partial groups never split.

The scheduler is transport-agnostic: ``submit(example, version) -> handle`` and ``poll(handle) -> rollouts | None`` are supplied by
the caller (HTTP client, in-process engine, or a test fake), so the policy logic is testable without a server.

Parity: surogate/grpo/orchestrator/scheduler.py:49-614.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional


@dataclass
class SchedulerConfig:
    batch_size: int = 64                 # rollouts per trainer step (ignored when token_batch_size is set)
    token_batch_size: Optional[int] = None
    group_size: int = 8
    max_inflight: int = 16               # group requests outstanding
    max_async_level: int = 2
    max_off_policy_steps: int = 4
    tasks_per_minute: Optional[float] = None   # cap on group requests issued per minute (rate-limited inference APIs)


@dataclass
class _Inflight:
    handle: Any
    example: Dict[str, Any]
    version: int
    server: int = 0


@dataclass
class _Ready:
    rollouts: List[Any]
    version: int
    tokens: int = 0


class RolloutScheduler:
    def __init__(self, cfg: SchedulerConfig, buffer, submit: Callable[[Dict[str, Any], int, int], Any], poll: Callable[[Any], Optional[List[Any]]],
                 cancel: Optional[Callable[[Any], None]] = None, num_servers: int = 1):
        self.cfg, self.buffer, self._submit, self._poll, self._cancel = cfg, buffer, submit, poll, cancel
        self.num_servers = max(1, num_servers)
        self.clock: Optional[Callable[[], float]] = None   # seconds; tests inject one, the default is time.monotonic
        self.inflight: List[_Inflight] = []
        self.ready: List[_Ready] = []
        self.requeued: List[Dict[str, Any]] = []
        self.trainer_version = 0
        self.depth_cap: Optional[int] = None
        self.sampling: Dict[str, Any] = {}
        self.cancelled = 0
        self._rr = 0
        self._off_policy_levels: List[int] = []

    # ------------------------------------------------------------------ knobs set by the orchestrator loop
    def set_depth_cap(self, cap: Optional[int]) -> None:
        self.depth_cap = cap

    def set_sampling_args(self, sampling: Dict[str, Any]) -> None:
        self.sampling = dict(sampling)

    @property
    def uses_token_batching(self) -> bool:
        return self.cfg.token_batch_size is not None

    @property
    def batch_target(self) -> int:
        return int(self.cfg.token_batch_size if self.uses_token_batching else self.cfg.batch_size)

    def may_issue(self, step: int) -> bool:
        return step - self.trainer_version <= self.cfg.max_async_level

    # ------------------------------------------------------------------ the two events
    def on_policy_update(self, version: int) -> int:
        """The trainer published ``version``: cancel what would be too stale when it finishes; returns the number cancelled."""
        self.trainer_version = version
        keep, dropped = [], 0
        for r in self.inflight:
            if version - r.version > self.cfg.max_off_policy_steps:
                if self._cancel is not None:
                    self._cancel(r.handle)
                self.requeued.append(r.example)
                dropped += 1
            else:
                keep.append(r)
        self.inflight = keep
        self.cancelled += dropped
        return dropped

    def _example_with_cap(self, ex: Dict[str, Any]) -> Dict[str, Any]:
        if self.depth_cap is None:
            return ex
        ex = dict(ex)
        info = dict(ex.get("info") or {})
        info["max_turns"] = min(int(info.get("max_turns", self.depth_cap)), self.depth_cap)
        ex["info"] = info
        return ex

    def fill(self, step: int) -> int:
        """Issue requests until ``max_inflight`` are outstanding (as long as generation may run at ``step``)."""
        issued = 0
        while len(self.inflight) < self.cfg.max_inflight and self.may_issue(step) and self._rate_allows():
            ex = self.requeued.pop(0) if self.requeued else (self.buffer.sample_examples(1) or [None])[0]
            if ex is None:
                break
            server = self._rr % self.num_servers   # round robin over inference servers
            self._rr += 1
            handle = self._submit(self._example_with_cap(ex), self.trainer_version, server)
            self.inflight.append(_Inflight(handle, ex, self.trainer_version, server))
            issued += 1
        return issued

    def _rate_allows(self) -> bool:
        """Token bucket for ``tasks_per_minute``: one token per request, refilled continuously, at most one minute's worth saved up."""
        rate = self.cfg.tasks_per_minute
        if not rate or rate <= 0:
            return True
        import time

        now = (self.clock or time.monotonic)()
        last = getattr(self, "_rate_last", None)
        tokens = getattr(self, "_rate_tokens", 1.0)
        if last is not None:
            tokens = min(float(rate), tokens + (now - last) * rate / 60.0)
        self._rate_last = now
        if tokens < 1.0:
            self._rate_tokens = tokens
            return False
        self._rate_tokens = tokens - 1.0
        return True

    def collect(self) -> int:
        """Move finished groups from in-flight to ready; returns how many finished."""
        done, still = 0, []
        for r in self.inflight:
            res = self._poll(r.handle)
            if res is None:
                still.append(r)
                continue
            for ro in res:
                ro.policy_version = r.version
                ro.meta.setdefault("example_id", r.example.get("example_id"))
                ro.meta.setdefault("task", r.example.get("task", "default"))
            self.ready.append(_Ready(list(res), r.version, sum(len(ro) for ro in res)))
            done += 1
        self.inflight = still
        return done

    # ------------------------------------------------------------------ batches
    def _progress(self) -> int:
        return sum(g.tokens if self.uses_token_batching else len(g.rollouts) for g in self.ready)

    def batch_ready(self) -> bool:
        return self._progress() >= self.batch_target

    def take_batch(self) -> List[List[Any]]:
        """Whole groups, oldest first, until the target is met; each rollout is tagged with its off-policy level."""
        out, got = [], 0
        while self.ready and got < self.batch_target:
            g = self.ready.pop(0)
            level = self.trainer_version - g.version
            for ro in g.rollouts:
                ro.meta["off_policy_level"] = level
            self._off_policy_levels.append(level)
            out.append(g.rollouts)
            got += g.tokens if self.uses_token_batching else len(g.rollouts)
        return out

    def metrics(self) -> Dict[str, float]:
        lv = self._off_policy_levels or [0]
        m = {"scheduler/inflight": float(len(self.inflight)), "scheduler/ready_groups": float(len(self.ready)), "scheduler/cancelled": float(self.cancelled),
             "scheduler/off_policy_max": float(max(lv)), "scheduler/off_policy_min": float(min(lv)), "scheduler/off_policy_mean": float(sum(lv) / len(lv)),
             "scheduler/async_level": float(self.cfg.max_async_level)}
        self._off_policy_levels = []
        return m

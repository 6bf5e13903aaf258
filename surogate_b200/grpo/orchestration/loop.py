"""Asynchronous orchestrator loop: the scheduler keeps group requests in flight on a thread pool while finished groups are
scored, filtered, turned into advantages and shipped to the trainer; the example buffer steers sampling away from prompts
without signal; the depth budget caps multi-turn episodes; progress and buffer pools are checkpointed for resume.

    while step < max_steps:
        scheduler.on_policy_update(version published by the trainer)
        scheduler.fill(step); scheduler.collect()
        if scheduler.batch_ready():
            groups  = scheduler.take_batch()
            filters -> advantages -> buffer.update(groups) -> pack -> transport.send(step)

Parity: surogate/grpo/orchestrator/grpo_orch.py:150-1011 (main loop), ckpt.py:26-119 (orchestrator checkpoints).
"""
from __future__ import annotations

import json
import os
import time
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

import numpy as np

from ..packer import Rollout, pack_rollouts
from .advantage import compute_advantages
from .buffer import BufferConfig, ExampleBuffer
from .depth import DepthObservation, RolloutDepthController
from .filters import apply_filters, make_filters
from .scheduler import RolloutScheduler, SchedulerConfig


@dataclass
class AsyncOrchestratorConfig:
    group_size: int = 8
    batch_size: int = 64                       # rollouts per trainer step
    token_batch_size: Optional[int] = None
    sequence_len: int = 2048
    rows_per_step: int = 8
    max_steps: int = 100
    max_inflight: int = 16
    max_async_level: int = 2
    max_off_policy_steps: int = 4
    workers: int = 16                          # threads that wait on the inference server
    advantage: str = "default"                 # default | std | module:function
    length_weighted_mean: bool = False
    filters: List[Dict[str, Any]] = field(default_factory=list)
    buffer: Dict[str, Any] = field(default_factory=dict)
    depth: Dict[str, Any] = field(default_factory=lambda: {"enabled": False})
    sampling: Dict[str, Any] = field(default_factory=lambda: {"max_tokens": 512, "temperature": 1.0})
    checkpoint_dir: Optional[str] = None
    checkpoint_every: int = 0
    keep_checkpoints: int = 2
    eval_every: int = 0                        # evaluate on ``eval_examples`` every this many steps (0 = never)
    eval_samples: int = 4
    eval_ks: Sequence[int] = (1, 4)
    eval_pass_threshold: float = 1.0
    temperature_schedule: Optional[Dict[str, Any]] = None   # {type: linear | cosine, start, end, total_steps}: sampling temperature by step
    tasks_per_minute: Optional[float] = None   # cap on group requests per minute
    val_every: int = 0                         # every this many steps: rollouts on ``val_examples`` training prompts, rewards logged, nothing trained
    val_examples: int = 16
    val_samples: int = 1
    metrics_file: Optional[str] = None         # every step's metrics as one JSON line (``dump_metrics``)
    poll_s: float = 0.01
    step_timeout_s: float = 3600.0
    vocab_size: int = 32000
    pad_token_id: int = 0


@dataclass
class Progress:
    step: int = 0
    total_tokens: int = 0
    total_samples: int = 0
    total_problems: int = 0


class OrchestratorCheckpoints:
    """``<dir>/step_N/{progress.json, buffer/*.jsonl}``; old steps are pruned."""

    def __init__(self, directory: str, keep: int = 2):
        self.dir, self.keep = directory, keep

    def path(self, step: int) -> str:
        return os.path.join(self.dir, f"step_{step}")

    def save(self, progress: Progress, buffer: ExampleBuffer) -> str:
        p = self.path(progress.step)
        os.makedirs(p, exist_ok=True)
        buffer.save(os.path.join(p, "buffer"))
        tmp = os.path.join(p, "progress.json.tmp")
        with open(tmp, "w") as f:
            json.dump(asdict(progress), f)
        os.replace(tmp, os.path.join(p, "progress.json"))
        import shutil

        for s in self.steps()[:-self.keep]:
            shutil.rmtree(self.path(s), ignore_errors=True)
        return p

    def steps(self) -> List[int]:
        if not os.path.isdir(self.dir):
            return []
        return sorted(int(d[5:]) for d in os.listdir(self.dir) if d.startswith("step_") and d[5:].isdigit()
                      and os.path.exists(os.path.join(self.dir, d, "progress.json")))

    def load_latest(self, buffer: ExampleBuffer) -> Optional[Progress]:
        steps = self.steps()
        if not steps:
            return None
        p = self.path(steps[-1])
        with open(os.path.join(p, "progress.json")) as f:
            prog = Progress(**json.load(f))
        buffer.load(os.path.join(p, "buffer"))
        return prog


class AsyncOrchestrator:
    """``generate_group(example, n, sampling, policy_version, server) -> [Rollout]`` does one prompt's group (single- or
    multi-turn) and sets each rollout's ``reward``; it runs on a worker thread.  ``policy_version()`` reads the newest version
    the trainer published; ``transport.send(step, arrays, meta)`` ships a packed batch."""

    def __init__(self, cfg: AsyncOrchestratorConfig, examples: Sequence[Dict[str, Any]], generate_group: Callable[..., List[Rollout]], transport,
                 policy_version: Callable[[], int], num_servers: int = 1, on_step: Optional[Callable[[Dict[str, float]], None]] = None,
                 eval_examples: Optional[Sequence[Dict[str, Any]]] = None, env_names: Optional[Sequence[str]] = None):
        self.cfg, self.transport, self.policy_version, self.on_step = cfg, transport, policy_version, on_step
        self.eval_examples, self.num_servers = list(eval_examples or []), max(1, num_servers)
        self.buffer = ExampleBuffer(examples, BufferConfig(**cfg.buffer), env_names)   # ``env_names`` fixes the order ``buffer.env_ratios`` refers to
        self.pool = ThreadPoolExecutor(max_workers=cfg.workers, thread_name_prefix="rollout")
        self.generate_group = generate_group
        sc = SchedulerConfig(batch_size=cfg.batch_size, token_batch_size=cfg.token_batch_size, group_size=cfg.group_size, max_inflight=cfg.max_inflight,
                             max_async_level=cfg.max_async_level, max_off_policy_steps=cfg.max_off_policy_steps, tasks_per_minute=cfg.tasks_per_minute)
        self.scheduler = RolloutScheduler(sc, self.buffer, self._submit, self._poll, self._cancel, num_servers)
        self.scheduler.set_sampling_args(cfg.sampling)
        self.filters = make_filters(cfg.filters, cfg.vocab_size)
        self.depth = RolloutDepthController(**cfg.depth)
        self.progress = Progress()
        self.ckpt = OrchestratorCheckpoints(cfg.checkpoint_dir, cfg.keep_checkpoints) if cfg.checkpoint_dir else None
        self.history: List[Dict[str, float]] = []

    # ------------------------------------------------------------------ scheduler transport: futures on the pool
    def _submit(self, example, version, server) -> Future:
        return self.pool.submit(self.generate_group, example, self.cfg.group_size, dict(self.scheduler.sampling), version, server)

    @staticmethod
    def _poll(fut: Future):
        return fut.result() if fut.done() else None

    @staticmethod
    def _cancel(fut: Future) -> None:
        fut.cancel()   # a request already on the wire finishes and is discarded

    # ------------------------------------------------------------------ one trainer batch
    def resume(self) -> int:
        if self.ckpt is not None:
            got = self.ckpt.load_latest(self.buffer)
            if got is not None:
                self.progress = got
        return self.progress.step

    def _score(self, groups: List[List[Rollout]]) -> Dict[str, float]:
        flat = [r for g in groups for r in g]
        stats = apply_filters(self.filters, flat)
        sizes = {len(g) for g in groups}
        if any("episode" in r.meta for r in flat):
            # multi-turn groups: an episode may have produced several samples; the advantage belongs to the episode
            adv = []
            for g in groups:
                order = sorted({r.meta.get("episode", i) for i, r in enumerate(g)})
                first = {k: next(r for i, r in enumerate(g) if r.meta.get("episode", i) == k) for k in order}
                length = {k: sum(len(r.completion_ids) for i, r in enumerate(g) if r.meta.get("episode", i) == k) for k in order}
                a = compute_advantages([first[k].reward for k in order], [length[k] for k in order], len(order), self.cfg.advantage,
                                       **({"length_weighted_mean": True} if self.cfg.length_weighted_mean and self.cfg.advantage == "default" else {}))
                by = dict(zip(order, a))
                adv += [by[r.meta.get("episode", i)] for i, r in enumerate(g)]
        elif len(sizes) == 1:
            n = sizes.pop()
            adv = compute_advantages([r.reward for r in flat], [len(r.completion_ids) for r in flat], n, self.cfg.advantage,
                                     **({"length_weighted_mean": True} if self.cfg.length_weighted_mean and self.cfg.advantage == "default" else {}))
        else:   # ragged groups (a request returned fewer completions): one group at a time
            adv = []
            for g in groups:
                adv += compute_advantages([r.reward for r in g], [len(r.completion_ids) for r in g], len(g), self.cfg.advantage)
        for r, a in zip(flat, adv):
            r.advantage = a
        rewards = np.array([r.reward for r in flat], dtype=np.float64) if flat else np.zeros(1)
        stats.update({"reward/mean": float(rewards.mean()), "reward/std": float(rewards.std()),
                      "completion_len/mean": float(np.mean([len(r.completion_ids) for r in flat])) if flat else 0.0})
        return stats

    def run_step(self, step: int) -> Dict[str, float]:
        t0 = time.time()
        s = self.scheduler
        self.buffer.reset_step_metrics()
        s.set_depth_cap(self.depth.cap_for_step(step))
        if self.cfg.temperature_schedule:
            from ..config_compat import temperature_at

            temp = temperature_at(step, self.cfg.temperature_schedule, self.cfg.max_steps)
            s.set_sampling_args(dict(self.cfg.sampling, temperature=temp))
        kept: List[Rollout] = []
        observations: List[DepthObservation] = []
        stats: Dict[str, float] = {}
        while True:
            s.on_policy_update(max(0, self.policy_version()))
            s.fill(step)
            s.collect()
            if s.batch_ready() or (not s.inflight and s.ready):
                groups = s.take_batch()
                stats = self._score(groups)
                for g in groups:
                    for r in g:
                        observations.append(DepthObservation(int(r.meta.get("turns", 1)), float(r.reward), bool(r.meta.get("truncated", False))))
                self.buffer.update(groups)
                want = self.cfg.batch_size if not s.uses_token_batching else len(self.buffer.rollouts)
                kept += self.buffer.sample_rollouts(want - len(kept) if not s.uses_token_batching else want)
                if (len(kept) >= self.cfg.batch_size and not s.uses_token_batching) or (s.uses_token_batching and sum(len(r) for r in kept) >= s.batch_target):
                    break
                if kept and not s.inflight and not s.ready and not s.may_issue(step):
                    break
            if time.time() - t0 > self.cfg.step_timeout_s:
                raise TimeoutError(f"step {step}: no full batch within {self.cfg.step_timeout_s}s ({len(kept)} rollouts with signal so far)")
            time.sleep(self.cfg.poll_s)
        self.depth.observe(step, observations)
        batches = pack_rollouts(kept, self.cfg.sequence_len, self.cfg.rows_per_step, self.cfg.pad_token_id)
        first = batches[0]
        meta = {"policy_version": min(r.policy_version for r in kept), "n_samples": first.n_samples, "reward_mean": stats.get("reward/mean", 0.0)}
        self.transport.send(step, first.arrays(), meta)
        self.progress.step = step + 1
        self.progress.total_samples += len(kept)
        self.progress.total_tokens += sum(len(r) for r in kept)
        self.progress.total_problems += len({r.meta.get("example_id") for r in kept})
        out = {"step": float(step), "time/step_s": time.time() - t0, **stats, **s.metrics(), **self.buffer.metrics(), **self.depth.metrics(),
               "progress/total_tokens": float(self.progress.total_tokens), "progress/total_samples": float(self.progress.total_samples)}
        if self.eval_examples and self.cfg.eval_every and (step + 1) % self.cfg.eval_every == 0:
            from .evaluation import evaluate_policy

            out.update(evaluate_policy(self.eval_examples, self.generate_group, self.cfg.eval_samples, self.cfg.sampling, max(0, self.policy_version()),
                                       self.cfg.eval_ks, self.cfg.eval_pass_threshold, self.num_servers))
        if self.cfg.val_every and (step + 1) % self.cfg.val_every == 0:
            out.update(self.validate())
        if self.cfg.metrics_file:
            os.makedirs(os.path.dirname(os.path.abspath(self.cfg.metrics_file)), exist_ok=True)
            with open(self.cfg.metrics_file, "a") as f:
                f.write(json.dumps(out, default=float) + "\n")
        if self.ckpt is not None and self.cfg.checkpoint_every and (step + 1) % self.cfg.checkpoint_every == 0:
            self.ckpt.save(self.progress, self.buffer)
        self.history.append(out)
        if self.on_step is not None:
            self.on_step(out)
        return out

    def validate(self) -> Dict[str, float]:
        """Rollouts on a fixed sample of the training prompts with the current policy: the reward trend on known prompts, outside
        the training batches (no pools are updated, nothing is sent to the trainer)."""
        from .evaluation import evaluate_policy

        pool = [e for name in self.buffer.pools.values() for env in name.values() for e in env.values()]
        pool.sort(key=lambda e: e.get("example_id", 0))
        sample = pool[:max(1, self.cfg.val_examples)]
        res = evaluate_policy(sample, self.generate_group, self.cfg.val_samples, self.cfg.sampling, max(0, self.policy_version()), (1,), self.cfg.eval_pass_threshold,
                              self.num_servers)
        return {k.replace("eval/", "val/"): v for k, v in res.items()}

    def run(self) -> List[Dict[str, float]]:
        try:
            for step in range(self.resume(), self.cfg.max_steps):
                self.run_step(step)
        finally:
            self.pool.shutdown(wait=False, cancel_futures=True)
        return self.history


# ------------------------------------------------------------------------------------------ wiring to the synchronous orchestrator's parts


def make_generate_group(orch) -> Callable[..., List[Rollout]]:
    """``generate_group`` for ``AsyncOrchestrator`` built from a configured ``grpo.orchestrator.Orchestrator`` (tokenizer, inference
    client(s), reward function or environment): one prompt's group, single- or multi-turn, rewards set, advantages left to the loop.
    ``orch.client`` may be a list of clients (one per inference server): the scheduler's ``server`` index picks one."""
    from ..orchestrator import Orchestrator  # noqa: F401  (type only)

    def pick(server: int):
        c = orch.client
        return c[server % len(c)] if isinstance(c, (list, tuple)) else c

    def generate_group(example, n, sampling, version, server):
        env = orch.env_for(example) if hasattr(orch, "env_for") else orch.env
        out: List[Rollout] = []
        if env is not None and hasattr(env, "env_response"):
            # everything an episode needs travels as arguments: this function runs on several worker threads at once
            cap = (example.get("info") or {}).get("max_turns")
            eps = orch.multi_turn_group(example, sampling, env=env, client=pick(server), group_size=n, max_turns=cap)
            depth: Dict[int, int] = {}
            for _, _, _, mask, _, k in eps:   # turns of an episode = policy spans over all of its samples
                depth[k] = depth.get(k, 0) + (1 + sum(1 for a, b in zip(mask, mask[1:]) if a == 0 and b == 1) if mask else 0)
            for pids, ids, lps, mask, r, k in eps:
                if ids:
                    turns = depth[k]
                    out.append(Rollout(pids, ids, lps, 0.0, float(r), version, 0, {"turns": turns, "truncated": cap is not None and turns >= int(cap), "episode": k},
                                       completion_mask=mask))
            if getattr(orch, "teacher", None) is not None:
                orch.teacher.score(out)
            return out
        pids = orch._prompt_ids(example)
        gens = pick(server).generate(pids, n, sampling)
        rewards = [float(r) for r in orch.reward_fn(example, [t for _, _, t in gens])]
        if orch.cfg.length_penalty:
            rewards = [r - orch.cfg.length_penalty * len(ids) for r, (ids, _, _) in zip(rewards, gens)]
        for (ids, lps, _), r in zip(gens, rewards):
            if ids and len(lps) == len(ids):
                out.append(Rollout(pids, ids, lps, 0.0, r, version, 0, {"turns": 1}))
        if getattr(orch, "teacher", None) is not None:
            orch.teacher.score(out)
        return out

    return generate_group


def async_config_from(cfg, raw: Optional[Dict[str, Any]] = None, vocab_size: int = 32000, pad_token_id: int = 0) -> AsyncOrchestratorConfig:
    """``OrchestratorConfig`` (+ the raw YAML dict for the keys only the asynchronous loop knows) -> ``AsyncOrchestratorConfig``."""
    raw = raw or {}
    a = AsyncOrchestratorConfig(group_size=cfg.group_size, batch_size=int(raw.get("batch_size", cfg.group_size * cfg.prompts_per_step)),
                                token_batch_size=raw.get("token_batch_size"), sequence_len=cfg.sequence_len, rows_per_step=cfg.rows_per_step,
                                max_steps=cfg.max_steps, max_inflight=int(raw.get("max_inflight", 2 * cfg.prompts_per_step)), max_async_level=cfg.max_async_level,
                                max_off_policy_steps=int(raw.get("max_off_policy_steps", 4)), workers=int(raw.get("workers", 2 * cfg.prompts_per_step)),
                                advantage=str(raw.get("advantage", "default")), length_weighted_mean=bool(raw.get("length_weighted_mean", False)),
                                filters=list(raw.get("filters", [])), buffer=dict(raw.get("buffer", {"seed": cfg.seed, "online_difficulty_filtering": cfg.filter_zero_advantage})),
                                depth=dict(raw.get("depth", {"enabled": False})),
                                sampling={"max_tokens": cfg.max_tokens, "temperature": cfg.temperature, "top_p": cfg.top_p, **cfg.extra_sampling},
                                checkpoint_dir=raw.get("checkpoint_dir"), checkpoint_every=int(raw.get("checkpoint_every", 0)),
                                keep_checkpoints=int(raw.get("keep_checkpoints", 2)), eval_every=int(raw.get("eval_every", 0)), eval_samples=int(raw.get("eval_samples", 4)),
                                temperature_schedule=raw.get("temperature_schedule"), tasks_per_minute=raw.get("tasks_per_minute"),
                                val_every=int(raw.get("val_every", 0)), val_examples=int(raw.get("val_examples", 16)), val_samples=int(raw.get("val_samples", 1)),
                                metrics_file=raw.get("metrics_file"), vocab_size=vocab_size, pad_token_id=pad_token_id)
    return a

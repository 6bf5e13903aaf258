"""GRPO orchestrator: prompts -> rollouts from an OpenAI-compatible inference server -> rewards -> group advantages ->
packed batches -> transport to the trainer, kept at most ``max_async_level`` policy versions ahead of the trainer.

The inference client is an interface (``generate(prompt_ids | messages, n, sampling) -> [(token_ids, logprobs, text)]``);
``OpenAIClient`` talks to vLLM's ``/v1/completions`` with ``logprobs`` and ``return_token_ids``; tests inject a fake.
The depth controller blocks generation of step ``s`` until the trainer has published policy version
``s - max_async_level`` — rollouts are never more than that many updates stale, and their recorded
``policy_version`` lets the trainer's ratio cap drop what is too far off-policy.

Parity: surogate/grpo/orchestrator/grpo_orch.py (rollout loop, buffer, scheduler, depth controller).
"""
from __future__ import annotations

import json
import time
import urllib.request
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .config import OrchestratorConfig
from .loss import group_advantages
from .packer import PackedBatch, Rollout, pack_rollouts
from .rewards import resolve_reward


class OpenAIClient:
    def __init__(self, base_url: str, model: str, timeout_s: float = 600.0, api_key: str = "EMPTY", headers: Optional[Dict[str, str]] = None):
        self.url, self.model, self.timeout, self.key = base_url.rstrip("/") + "/completions", model, timeout_s, api_key
        self.headers = dict(headers or {})

    def generate(self, prompt_ids: List[int], n: int, sampling: Dict[str, Any]) -> List[Tuple[List[int], List[float], str]]:
        body = {"model": self.model, "prompt": prompt_ids, "n": n, "logprobs": 1, "return_token_ids": True, **sampling}
        req = urllib.request.Request(self.url, data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json", "Authorization": f"Bearer {self.key}", **self.headers})
        with urllib.request.urlopen(req, timeout=self.timeout) as r:
            resp = json.loads(r.read())
        out = []
        for ch in resp["choices"]:
            lp = ch.get("logprobs") or {}
            ids = ch.get("token_ids") or []
            out.append((list(ids), [float(x) for x in (lp.get("token_logprobs") or [])], ch.get("text", "")))
        return out


class DepthController:
    """Keeps generation within ``max_async_level`` policy versions of the trainer."""

    def __init__(self, max_async_level: int, current_version: Callable[[], int], poll_s: float = 0.05, timeout_s: float = 3600.0):
        self.k, self.version, self.poll, self.timeout = max_async_level, current_version, poll_s, timeout_s

    def wait_until_allowed(self, step: int) -> int:
        t0 = time.time()
        while True:
            v = self.version()
            if step - v <= self.k:
                return v
            if time.time() - t0 > self.timeout:
                raise TimeoutError(f"trainer did not reach policy version {step - self.k} (at {v})")
            time.sleep(self.poll)


@dataclass
class StepStats:
    step: int
    reward_mean: float
    reward_std: float
    completion_len: float
    groups_kept: int
    groups_total: int
    policy_version: int
    rows: int


class Orchestrator:
    def __init__(self, cfg: OrchestratorConfig, tokenizer, client, transport, policy_version: Callable[[], int], reward_fn=None):
        self.cfg, self.tok, self.client, self.transport = cfg, tokenizer, client, transport
        self.env = None
        self.envs: Dict[str, Any] = {}          # task name -> environment, when several environments train together
        self.env_reward_fns: Dict[str, Callable] = {}
        if getattr(cfg, "environments", None) and reward_fn is None:
            from .environments import as_reward_fn, load_environment

            for spec in cfg.environments:
                name = spec.get("name") or str(spec["id"]).split("@")[0]
                if name in self.envs or name == "all":
                    raise ValueError(f"environment name '{name}' is {'reserved' if name == 'all' else 'used twice'}")
                env = load_environment(spec["id"], path=cfg.environments_path, import_path=spec.get("path") or None,
                                       **dict(spec.get("args") or {}, **(spec.get("extra_env_kwargs") or {})))
                self.envs[name] = env
                self.env_reward_fns[name] = getattr(env, "score_group", None) or as_reward_fn(env)
            self.env = next(iter(self.envs.values()))
            first = next(iter(self.env_reward_fns.values()))
            reward_fn = lambda row, completions: self.env_reward_fns.get(row.get("task"), first)(row, completions)  # noqa: E731
        elif cfg.environment and reward_fn is None:  # single-turn scoring of the sampled completions by the environment's rubric
            from .environments import as_reward_fn, load_environment

            self.env = load_environment(cfg.environment, path=cfg.environments_path, import_path=getattr(cfg, "environment_import_path", "") or None,
                                        **cfg.environment_args)
            base_fn = getattr(self.env, "score_group", None) or as_reward_fn(self.env)
            reward_fn = lambda row, completions: self.env_reward_fns.get(row.get("task"), base_fn)(row, completions)  # noqa: E731 - rows of evaluation-only environments carry their task
        self.reward_fn = reward_fn or resolve_reward(cfg.reward)
        self.judge = None
        self.teacher = None
        if getattr(cfg, "teacher", None):
            from .teacher import TeacherScorer

            self.teacher = TeacherScorer.from_config(cfg.teacher)
        if getattr(cfg, "ruler", None) and cfg.ruler.get("enabled"):
            self.set_judge(cfg.ruler)
        self.depth = DepthController(cfg.max_async_level, policy_version)
        self.rng = np.random.default_rng(cfg.seed)
        self.prompts: List[Dict[str, Any]] = []
        self.buffer: List[Rollout] = []
        self.history: List[StepStats] = []

    def set_judge(self, ruler, scorer=None) -> None:
        """Switch the LLM-judge group reward on (``ruler``: the config section; ``scorer``: a ready ``RulerScorer``).  Single-turn
        groups are judged through the reward function, multi-turn episodes with their whole conversation."""
        from .ruler import build_ruler

        self.judge = scorer or build_ruler(ruler)
        if self.judge is not None:
            self.reward_fn = self.judge.wrap_reward_fn(self.reward_fn)

    def add_eval_environments(self, specs: Sequence[Dict[str, Any]], default_examples: Optional[int] = None) -> List[Dict[str, Any]]:
        """Environments that are only evaluated on: registered under their names (so their examples are rolled out and scored by
        them) and returned as evaluation rows: the environment's evaluation split, or the head of its dataset."""
        from .environments import as_reward_fn, load_environment

        rows: List[Dict[str, Any]] = []
        for spec in specs:
            name = spec.get("name") or str(spec["id"]).split("@")[0]
            env = self.envs.get(name)
            if env is None:
                env = load_environment(spec["id"], path=self.cfg.environments_path, import_path=spec.get("path") or None, **dict(spec.get("args") or {}))
                if not self.envs and self.env is not None:   # a single training environment so far: keep it reachable by task name
                    self.envs[getattr(self.env, "env_id", "default")] = self.env
                self.envs[name] = env
                self.env_reward_fns[name] = getattr(env, "score_group", None) or as_reward_fn(env)
            data = list(env.eval_dataset or env.dataset)
            n = spec.get("num_examples") or default_examples
            data = data[:int(n)] if n and int(n) > 0 else data
            multi = hasattr(env, "env_response")
            rows += [dict(ex, task=name) if multi else dict(ex, prompt=env.initial_messages(ex), task=name) for ex in data]
        return rows

    def env_for(self, row: Dict[str, Any]):
        """The environment a prompt belongs to (its ``task``), or the only one."""
        return self.envs.get(row.get("task"), self.env) if self.envs else self.env

    def load_prompts(self, rows: Optional[Sequence[Dict[str, Any]]] = None) -> None:
        if rows is None and self.envs:
            rows = []
            for name, env in self.envs.items():
                multi = hasattr(env, "env_response")
                rows += [dict(ex, task=name) if multi else dict(ex, prompt=env.initial_messages(ex), task=name) for ex in env.dataset]
        if rows is None and self.env is not None:
            rows = [dict(ex, prompt=self.env.initial_messages(ex)) for ex in self.env.dataset] if not hasattr(self.env, "env_response") else list(self.env.dataset)
        if rows is None:
            with open(self.cfg.prompts) as f:
                rows = [json.loads(l) for l in f if l.strip()]
        self.prompts = list(rows)

    def _prompt_ids(self, row: Dict[str, Any]) -> List[int]:
        p = row["prompt"]
        if isinstance(p, list):
            return self.tok.apply_chat_template_and_encode(p, add_generation_prompt=True)
        return self.tok.apply_chat_template_and_encode([{"role": "user", "content": str(p)}], add_generation_prompt=True)

    def multi_turn_group(self, row: Dict[str, Any], sampling: Dict[str, Any], env=None, client=None, group_size: Optional[int] = None, max_turns: Optional[int] = None):
        """``group_size`` episodes of a multi-turn environment for one example.  Each episode alternates a sampled assistant turn
        and the environment's reply; the conversation is re-encoded with the chat template after every reply and the tokens
        it added (end-of-turn marker, tool message, next generation prompt) join the sequence as context that is not trained
        on.  When re-encoding does not reproduce the tokens sampled so far (a template that rewrites earlier turns, e.g. drops
        old reasoning), the sample is closed there and the episode goes on in a NEW sample whose prompt is the re-encoded
        conversation, so no turn is lost: an episode yields one sample while the extension property holds and up to one per
        turn when it never does.  All samples of an episode carry its reward.
        Returns [(prompt_ids, token_ids, logprobs, mask, reward, episode_index)], one or more entries per episode."""
        env = env or self.env_for(row)
        client = client or self.client
        turn_cap = min(int(env.max_turns), int(max_turns)) if max_turns is not None else env.max_turns
        out = []
        conversations = []
        for _ in range(group_size or self.cfg.group_size):
            msgs = env.initial_messages(row)
            state = dict(env.setup_state(row), example=row)
            prompt0 = self.tok.apply_chat_template_and_encode(msgs, add_generation_prompt=True)
            ctx, comp, lps, mask, text, turns = list(prompt0), [], [], [], "", 0
            segments = []     # samples of this episode that were closed because the extension property broke
            while turns < turn_cap and len(ctx) < self.cfg.sequence_len:
                ids, lp, text = client.generate(ctx, 1, sampling)[0]
                if not ids or len(lp) != len(ids):
                    break
                comp += ids
                lps += lp
                mask += [1] * len(ids)
                msgs = msgs + [{"role": "assistant", "content": text}]
                turns += 1
                if env.is_completed(msgs, state):
                    break
                msgs = msgs + env.env_response(msgs, state)
                new_ctx = self.tok.apply_chat_template_and_encode(msgs, add_generation_prompt=True)
                full = prompt0 + comp
                if new_ctx[:len(full)] != full:   # the template rewrote what came before: close this sample, go on in a new one
                    segments.append((prompt0, comp, lps, mask))
                    prompt0, comp, lps, mask, ctx = list(new_ctx), [], [], [], new_ctx
                    continue
                extra = new_ctx[len(full):]
                comp += extra
                lps += [0.0] * len(extra)
                mask += [0] * len(extra)
                ctx = new_ctx
            reward, _ = env.score(row, dict(state, messages=msgs, completion=text, turns=turns))
            episode = len(conversations)
            for seg in segments + ([(prompt0, comp, lps, mask)] if comp or not segments else []):
                out.append(seg + (float(reward), episode))
            conversations.append(msgs)
        if self.judge is not None and out:
            first = {}
            for o in out:
                first.setdefault(o[5], o[4])
            judged, _ = self.judge.apply(conversations, [first[e] for e in range(len(conversations))])
            out = [o[:4] + (float(judged[o[5]]), o[5]) for o in out]
        return out

    def collect(self, step: int, version: int) -> Tuple[List[Rollout], Dict[str, float]]:
        c = self.cfg
        idx = self.rng.choice(len(self.prompts), size=min(c.prompts_per_step, len(self.prompts)), replace=False)
        sampling = {"max_tokens": c.max_tokens, "temperature": c.temperature, "top_p": c.top_p, **c.extra_sampling}
        rollouts: List[Rollout] = []
        rewards_all, lens, kept = [], [], 0
        for g, i in enumerate(idx):
            row = self.prompts[int(i)]
            if self.env_for(row) is not None and hasattr(self.env_for(row), "env_response"):  # multi-turn environment: episodes instead of single completions
                eps = self.multi_turn_group(row, sampling)
                by_episode = {}
                for e in eps:
                    by_episode.setdefault(e[5], e[4])
                rewards = [by_episode[k] for k in sorted(by_episode)]          # one reward per episode, however many samples it produced
                rewards_all += rewards
                lens += [sum(sum(e[3]) for e in eps if e[5] == k) for k in sorted(by_episode)]
                adv_by_episode = dict(zip(sorted(by_episode), group_advantages(torch.tensor(rewards), len(rewards), c.advantage_std_eps).tolist()))
                if c.filter_zero_advantage and max(rewards) - min(rewards) < 1e-12:
                    continue
                kept += 1
                for (pids, ids, lps, mask, r, k) in eps:
                    a = adv_by_episode[k]
                    if ids:
                        rollouts.append(Rollout(pids, ids, lps, a, r, version, g, completion_mask=mask))
                continue
            pids = self._prompt_ids(row)
            gens = self.client.generate(pids, c.group_size, sampling)
            rewards = [float(r) for r in self.reward_fn(row, [t for _, _, t in gens])]
            if c.length_penalty:
                rewards = [r - c.length_penalty * len(ids) for r, (ids, _, _) in zip(rewards, gens)]
            rewards_all += rewards
            lens += [len(ids) for ids, _, _ in gens]
            adv = group_advantages(torch.tensor(rewards), len(rewards), c.advantage_std_eps).tolist()
            if c.filter_zero_advantage and max(rewards) - min(rewards) < 1e-12:
                continue
            kept += 1
            for (ids, lps, _), a, r in zip(gens, adv, rewards):
                if ids and len(lps) == len(ids):
                    rollouts.append(Rollout(pids, ids, lps, a, r, version, g))
        if self.teacher is not None:
            self.teacher.score(rollouts)
        stats = {"reward_mean": float(np.mean(rewards_all)) if rewards_all else 0.0, "reward_std": float(np.std(rewards_all)) if rewards_all else 0.0,
                 "completion_len": float(np.mean(lens)) if lens else 0.0, "groups_kept": kept, "groups_total": len(idx)}
        return rollouts, stats

    def run_step(self, step: int) -> StepStats:
        version = self.depth.wait_until_allowed(step)
        need_rows = self.cfg.rows_per_step
        stats: Dict[str, float] = {}
        attempts = 0
        batches: List[PackedBatch] = []
        while not batches or batches[0].n_samples == 0:
            rollouts, stats = self.collect(step, version)
            self.buffer += rollouts
            batches = pack_rollouts(self.buffer, self.cfg.sequence_len, need_rows, self.tok.pad_token_id if self.tok.pad_token_id >= 0 else 0)
            attempts += 1
            if attempts > 16:
                raise RuntimeError("no rollout group with a reward spread after 16 attempts: the reward function gives no signal")
        first = batches[0]
        self.buffer = []  # what did not fit into the first batch is dropped rather than trained on stale
        self.transport.send(step, first.arrays(), {"policy_version": first.policy_version, "n_samples": first.n_samples, **stats})
        st = StepStats(step, stats["reward_mean"], stats["reward_std"], stats["completion_len"], int(stats["groups_kept"]), int(stats["groups_total"]),
                       version, need_rows)
        self.history.append(st)
        return st

    def run(self, start_step: int = 0) -> List[StepStats]:
        for step in range(start_step, self.cfg.max_steps):
            self.run_step(step)
            if hasattr(self.transport, "acked"):
                self.transport.cleanup(self.transport.acked() - 1)
        return self.history

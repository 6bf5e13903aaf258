"""A small, dependency-free environment layer for RL training and evaluation.

An environment owns a dataset of examples (``prompt`` = chat messages, ``answer``, free-form ``info``), knows how to run a
rollout against a *policy* (any callable ``messages -> assistant text``: an OpenAI-compatible endpoint, a local model, a
stub) and scores the result with a rubric of weighted reward functions.  Single-turn environments ask once; multi-turn ones
loop ``policy -> env_response`` until the environment says the episode is over or ``max_turns`` is reached.

``as_reward_fn(env)`` adapts an environment to the ``reward_fn(row, completions) -> scores`` hook of the GRPO orchestrator;
``evaluate`` is what ``surogate vf-eval`` runs.

Parity: the reference builds its environments on the ``verifiers`` package (environments/*/ *.py, surogate/cli/vf_eval.py);
this is the subset of that interface they use.
"""
from __future__ import annotations

import importlib
import json
import statistics
import urllib.request
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

Messages = List[Dict[str, str]]
Policy = Callable[[Messages], str]
RewardFn = Callable[..., float]


class Rubric:
    def __init__(self, funcs: Sequence[RewardFn], weights: Optional[Sequence[float]] = None):
        self.funcs = list(funcs)
        self.weights = list(weights) if weights is not None else [1.0] * len(self.funcs)
        if len(self.weights) != len(self.funcs):
            raise ValueError("one weight per reward function")

    def score(self, **kw) -> Tuple[float, Dict[str, float]]:
        parts = {f.__name__: float(f(**kw)) for f in self.funcs}
        return sum(w * parts[f.__name__] for f, w in zip(self.funcs, self.weights)), parts


class Environment:
    env_id = "environment"

    def __init__(self, dataset: Sequence[Dict[str, Any]], rubric: Rubric, eval_dataset: Optional[Sequence[Dict[str, Any]]] = None,
                 system_prompt: str = ""):
        self.dataset, self.eval_dataset, self.rubric, self.system_prompt = list(dataset), list(eval_dataset or []), rubric, system_prompt

    def initial_messages(self, example: Dict[str, Any]) -> Messages:
        msgs = list(example["prompt"]) if isinstance(example["prompt"], list) else [{"role": "user", "content": str(example["prompt"])}]
        if self.system_prompt and (not msgs or msgs[0]["role"] != "system"):
            msgs = [{"role": "system", "content": self.system_prompt}] + msgs
        return msgs

    def rollout(self, policy: Policy, example: Dict[str, Any]) -> Dict[str, Any]:
        msgs = self.initial_messages(example)
        text = policy(msgs)
        return {"messages": msgs + [{"role": "assistant", "content": text}], "completion": text, "turns": 1}

    def score(self, example: Dict[str, Any], state: Dict[str, Any]) -> Tuple[float, Dict[str, float]]:
        return self.rubric.score(completion=state["completion"], answer=example.get("answer"), info=example.get("info", {}), state=state,
                                 prompt=example["prompt"])


class SingleTurnEnv(Environment):
    pass


class MultiTurnEnv(Environment):
    def __init__(self, *a, max_turns: int = 8, **kw):
        super().__init__(*a, **kw)
        self.max_turns = max_turns

    def setup_state(self, example: Dict[str, Any]) -> Dict[str, Any]:
        return {}

    def is_completed(self, messages: Messages, state: Dict[str, Any]) -> bool:
        raise NotImplementedError

    def env_response(self, messages: Messages, state: Dict[str, Any]) -> Messages:
        raise NotImplementedError

    def rollout(self, policy: Policy, example: Dict[str, Any]) -> Dict[str, Any]:
        msgs = self.initial_messages(example)
        state = dict(self.setup_state(example), example=example)
        turns, text = 0, ""
        while turns < self.max_turns:
            text = policy(msgs)
            msgs = msgs + [{"role": "assistant", "content": text}]
            turns += 1
            if self.is_completed(msgs, state):
                break
            msgs = msgs + self.env_response(msgs, state)
        return dict(state, messages=msgs, completion=text, turns=turns)


# ---------------------------------------------------------------------------------------------- policies
def openai_policy(base_url: str, model: str, temperature: Optional[float] = 0.7, max_tokens: Optional[int] = 1024, api_key: str = "EMPTY",
                  timeout_s: float = 300.0, headers: Optional[Dict[str, str]] = None, sampling_args: Optional[Dict[str, Any]] = None,
                  max_retries: int = 0) -> Policy:
    """Chat-completions endpoint (vLLM, or any OpenAI-compatible server) as a policy.  ``sampling_args`` are merged into the request
    body (``top_p``, ``stop``, ...); ``temperature`` / ``max_tokens`` of None leave the server's defaults; a failed request is
    retried ``max_retries`` times with back-off."""
    import time

    def call(messages: Messages) -> str:
        body: Dict[str, Any] = {"model": model, "messages": messages}
        if temperature is not None:
            body["temperature"] = temperature
        if max_tokens is not None:
            body["max_tokens"] = max_tokens
        body.update(sampling_args or {})
        req = urllib.request.Request(base_url.rstrip("/") + "/chat/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json", "Authorization": f"Bearer {api_key}", **(headers or {})})
        for attempt in range(max_retries + 1):
            try:
                with urllib.request.urlopen(req, timeout=timeout_s) as r:
                    return json.loads(r.read())["choices"][0]["message"]["content"] or ""
            except Exception:  # noqa: BLE001 - connection reset, 5xx, malformed body: retried alike
                if attempt == max_retries:
                    raise
                time.sleep(min(0.1 * 2.0 ** attempt, 5.0))
        return ""

    return call


# ---------------------------------------------------------------------------------------------- registry / evaluation
BUILTIN = {"markdown-table-qa": "surogate_b200.grpo.environments.markdown_table_qa", "multihop-tools": "surogate_b200.grpo.environments.multihop_tools",
           "ruler-task": "surogate_b200.grpo.environments.ruler_task"}


def load_environment(env_id: str, path: Optional[str] = None, import_path: Optional[str] = None, **kwargs) -> Environment:
    """Built-in id, a module ``<path>/<env_id with _>/<env_id with _>.py`` (what ``vf-init`` scaffolds), or (``import_path``: a
    directory put in front of ``sys.path``) an importable package named after the id, each exposing ``load_environment(**kwargs)``."""
    key = env_id.replace("_", "-")
    if key in BUILTIN:
        return importlib.import_module(BUILTIN[key]).load_environment(**kwargs)
    import os
    from importlib import util as importlib_util

    mod_name = env_id.replace("-", "_")
    if import_path:
        import sys

        if import_path not in sys.path:
            sys.path.insert(0, import_path)
        return importlib.import_module(mod_name).load_environment(**kwargs)
    for cand in (os.path.join(path or "./environments", mod_name, mod_name + ".py"), os.path.join(path or "./environments", key, mod_name + ".py")):
        if os.path.exists(cand):
            spec = importlib_util.spec_from_file_location(mod_name, cand)
            mod = importlib_util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            return mod.load_environment(**kwargs)
    raise KeyError(f"unknown environment '{env_id}' (built in: {sorted(BUILTIN)}; looked under {path or './environments'})")


def evaluate(env: Environment, policy: Policy, num_examples: int = 20, rollouts_per_example: int = 1, use_eval_split: bool = True,
             max_concurrent: int = 1, on_sample: Optional[Callable[[Dict[str, Any]], None]] = None) -> Dict[str, Any]:
    """Roll the policy out on the first ``num_examples`` examples (``rollouts_per_example`` times each), at most
    ``max_concurrent`` rollouts in flight; results keep the order of the examples whatever order they finish in."""
    data = (env.eval_dataset if (use_eval_split and env.eval_dataset) else env.dataset)[:num_examples]
    rewards: List[float] = []
    parts: Dict[str, List[float]] = {}
    samples = []
    jobs = [ex for ex in data for _ in range(rollouts_per_example)]

    def one(ex):
        state = env.rollout(policy, ex)
        total, p = env.score(ex, state)
        return ex, state, total, p

    if max_concurrent > 1 and len(jobs) > 1:
        from concurrent.futures import ThreadPoolExecutor

        with ThreadPoolExecutor(max_workers=min(max_concurrent, len(jobs))) as pool:
            results = list(pool.map(one, jobs))
    else:
        results = [one(ex) for ex in jobs]
    for ex, state, total, p in results:
        rewards.append(total)
        for k, v in p.items():
            parts.setdefault(k, []).append(v)
        samples.append({"answer": ex.get("answer"), "completion": state["completion"], "reward": total, "turns": state.get("turns", 1)})
        if on_sample is not None:
            on_sample(samples[-1])
    return {"env": env.env_id, "n": len(rewards), "mean_reward": statistics.fmean(rewards) if rewards else 0.0,
            "std_reward": statistics.pstdev(rewards) if len(rewards) > 1 else 0.0, "metrics": {k: statistics.fmean(v) for k, v in parts.items()},
            "samples": samples}


def as_reward_fn(env: Environment) -> Callable[[Dict[str, Any], List[str]], List[float]]:
    """Single-turn scoring of already generated completions (the GRPO orchestrator's ``reward_fn`` hook)."""

    def fn(row: Dict[str, Any], completions: List[str]) -> List[float]:
        return [env.score(row, {"completion": c, "messages": [], "turns": 1})[0] for c in completions]

    return fn

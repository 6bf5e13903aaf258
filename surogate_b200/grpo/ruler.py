"""Relative LLM-judge rewards for a group of trajectories ("RULER": relative universal LLM-elicited rewards).

All trajectories of one prompt go to an OpenAI-compatible judge in ONE request; the judge returns a score in [0, 1] per trajectory,
relative to the others of the group, which is exactly the signal a group-relative advantage needs, with no task-specific reward
code.  The shared beginning of the trajectories (system prompt, task) is sent once as context, each trajectory then only carries
what differs.

    mode: replace   reward = weight * judge score            (the environment's own reward is dropped)
          add       reward = environment reward + weight * judge score
          metric    reward unchanged; the judge score is only logged

``JudgePool`` spreads requests over several judge endpoints round robin under one concurrency cap, retries transport errors with
back-off and waits for the endpoints to come up.  A reply that cannot be parsed is asked for again (``max_retries_on_parse_error``);
when the judge still fails, ``swallow_exceptions`` decides between scoring the group 0 (and counting the failure) and raising.
Token usage is accumulated and priced when ``cost`` gives prices per million tokens.

Parity: surogate/rewards/ruler.py (RulerRubric, JudgeClientPool, build_ruler_rubric), surogate/core/config/grpo_orch_config.py:522-660.
"""
from __future__ import annotations

import itertools
import json
import os
import re
import threading
import time
import urllib.error
import urllib.request
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

DEFAULT_RUBRIC = """- A trajectory that reaches its goal always scores clearly higher than one that does not.
- Of two trajectories that reach the goal, the one that gets there with fewer detours, redundant tool calls or wasted reasoning scores higher.
- Small differences in quality give small differences in score, large differences give large ones.
- Meaningful progress without completion earns partial credit.
- Hallucinated facts, ignoring the request, or breaking explicit constraints of the system prompt lower the score."""

Messages = List[Dict[str, Any]]


class RulerJudgeError(RuntimeError):
    pass


@dataclass
class RulerConfig:
    enabled: bool = False
    mode: str = "replace"                    # replace | add | metric
    judge_model: Optional[str] = None
    judge: Dict[str, Any] = field(default_factory=dict)   # base_url (str | list), api_key_var, timeout, max_retries, headers
    rubric: Optional[str] = None
    weight: float = 1.0
    max_concurrent_judges: int = 32
    request_timeout: Optional[float] = None
    max_retries_on_parse_error: int = 2
    swallow_exceptions: bool = True
    debug: bool = False
    extra_body: Dict[str, Any] = field(default_factory=dict)
    sampling: Dict[str, Any] = field(default_factory=dict)
    cost: Optional[Dict[str, Any]] = None    # input_per_million, output_per_million

    def __post_init__(self):
        if self.mode not in ("replace", "add", "metric"):
            raise ValueError(f"ruler.mode must be replace, add or metric, got {self.mode!r}")
        if self.enabled and not self.judge_model:
            raise ValueError("ruler.enabled needs ruler.judge_model")

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> "RulerConfig":
        d = dict(d or {})
        known = set(cls.__dataclass_fields__)
        unknown = sorted(k for k in d if k not in known)
        if unknown:
            raise ValueError(f"unknown ruler key(s): {unknown}")
        return cls(**d)


class JudgePool:
    def __init__(self, base_urls: Sequence[str], api_key: str = "EMPTY", timeout_s: float = 120.0, max_concurrent: int = 32, max_retries: int = 4,
                 headers: Optional[Dict[str, str]] = None, opener: Optional[Callable[..., Any]] = None):
        if not base_urls:
            raise ValueError("the judge needs at least one base_url")
        self.urls = [u.rstrip("/") for u in base_urls]
        self.key, self.timeout, self.max_retries, self.headers = api_key, timeout_s, max_retries, dict(headers or {})
        self._next = itertools.cycle(range(len(self.urls)))
        self._lock = threading.Lock()
        self._slots = threading.Semaphore(max(1, max_concurrent))
        self._open = opener or urllib.request.urlopen
        self.requests = 0

    @classmethod
    def from_config(cls, cfg: RulerConfig, **kw) -> "JudgePool":
        j = cfg.judge or {}
        urls = j.get("base_url") or ["http://localhost:8001/v1"]
        urls = [urls] if isinstance(urls, str) else list(urls)
        var = j.get("api_key_var", "RULER_JUDGE_API_KEY")
        return cls(urls, (os.environ.get(var) if var else None) or "EMPTY", float(cfg.request_timeout or j.get("timeout") or 120.0), cfg.max_concurrent_judges,
                   int(j.get("max_retries", 4)), j.get("headers"), **kw)

    def _pick(self) -> str:
        with self._lock:
            return self.urls[next(self._next)]

    def chat(self, body: Dict[str, Any]) -> Dict[str, Any]:
        """One chat-completions request on the next endpoint; transport errors and 5xx / 429 replies are retried on the following
        endpoint with back-off."""
        last: Optional[BaseException] = None
        with self._slots:
            for attempt in range(self.max_retries + 1):
                url = self._pick() + "/chat/completions"
                req = urllib.request.Request(url, data=json.dumps(body).encode(),
                                             headers={"Content-Type": "application/json", "Authorization": f"Bearer {self.key}", **self.headers})
                try:
                    with self._lock:
                        self.requests += 1
                    with self._open(req, timeout=self.timeout) as r:
                        return json.loads(r.read())
                except urllib.error.HTTPError as e:
                    if e.code < 500 and e.code != 429:
                        raise RulerJudgeError(f"judge at {url} answered {e.code}") from e
                    last = e
                except Exception as e:  # noqa: BLE001 - connection refused / reset / timeout / damaged body: all retried
                    last = e
                time.sleep(min(0.05 * 2.0 ** attempt, 5.0))
        raise RulerJudgeError(f"judge unreachable after {self.max_retries + 1} attempts: {last}")

    def wait_for_ready(self, timeout_s: float = 600.0, poll_s: float = 2.0) -> None:
        """Block until every endpoint answers ``GET /models`` (a judge engine started next to the run needs a while to load)."""
        deadline = time.time() + timeout_s
        for url in self.urls:
            while True:
                try:
                    with self._open(urllib.request.Request(url + "/models", headers={"Authorization": f"Bearer {self.key}", **self.headers}), timeout=10.0) as r:
                        r.read()
                    break
                except Exception as e:  # noqa: BLE001
                    if time.time() > deadline:
                        raise RulerJudgeError(f"judge at {url} did not come up within {timeout_s:.0f}s: {e}") from e
                    time.sleep(poll_s)


def common_prefix_len(trajectories: Sequence[Messages]) -> int:
    """Number of leading messages that are identical in every trajectory."""
    if not trajectories:
        return 0
    keyed = [[json.dumps(m, sort_keys=True, default=str) for m in t] for t in trajectories]
    n = 0
    for column in zip(*keyed):
        if any(c != column[0] for c in column):
            break
        n += 1
    return min(n, min(len(t) for t in keyed))


def parse_scores(text: str, n: int) -> List[float]:
    """Scores in trajectory order from the judge's reply: ``{"scores": [{"trajectory_id": "1", "score": 0.7, ...}, ...]}`` in any
    order, or a plain list of numbers.  Raises ``ValueError`` when the reply does not cover the ``n`` trajectories."""
    m = re.search(r"\{.*\}", text or "", re.S)
    if not m:
        raise ValueError("no JSON object in the judge's reply")
    obj = json.loads(m.group(0))
    entries = obj.get("scores")
    if not isinstance(entries, list):
        raise ValueError("the reply has no `scores` list")
    if entries and all(isinstance(e, (int, float)) for e in entries):
        if len(entries) != n:
            raise ValueError(f"{len(entries)} scores for {n} trajectories")
        return [min(1.0, max(0.0, float(e))) for e in entries]
    by_id: Dict[int, float] = {}
    for e in entries:
        if not isinstance(e, dict) or "score" not in e:
            raise ValueError("a score entry is not an object with `score`")
        ident = re.sub(r"\D", "", str(e.get("trajectory_id", "")))
        if ident == "":
            raise ValueError("a score entry has no trajectory_id")
        by_id[int(ident)] = min(1.0, max(0.0, float(e["score"])))
    if sorted(by_id) != list(range(1, n + 1)):
        raise ValueError(f"scores for trajectories {sorted(by_id)}, expected 1..{n}")
    return [by_id[i] for i in range(1, n + 1)]


class RulerScorer:
    def __init__(self, cfg: RulerConfig, pool: JudgePool):
        self.cfg, self.pool = cfg, pool
        self.rubric = (cfg.rubric or DEFAULT_RUBRIC).strip()
        self._lock = threading.Lock()
        self.groups = self.failures = self.parse_retries = 0
        self.input_tokens = self.output_tokens = 0

    # -- request
    def build_messages(self, trajectories: Sequence[Messages]) -> Messages:
        shared = common_prefix_len(trajectories)
        context = trajectories[0][:shared] if trajectories else []
        parts = []
        if context:
            parts.append("<context>\n" + "\n".join(json.dumps(m, default=str) for m in context) + "\n</context>")
        for i, t in enumerate(trajectories, 1):
            parts.append(f'<trajectory id="{i}">\n' + "\n".join(json.dumps(m, default=str) for m in t[shared:]) + "\n</trajectory>")
        system = ("All of the trajectories below were given the same goal. Score each of them between 0 and 1 relative to the others, "
                  "taking into account how well it achieves the goal.\n\nGrading standards:\n" + self.rubric +
                  '\n\nReply with JSON only: {"scores": [{"trajectory_id": "<id>", "explanation": "<one or two sentences>", "score": <0..1>}, ...]} '
                  "with one entry per trajectory.")
        return [{"role": "system", "content": system}, {"role": "user", "content": "\n\n".join(parts)}]

    def score_group(self, trajectories: Sequence[Messages]) -> Optional[List[float]]:
        """Judge scores in trajectory order, or None when the judge failed and ``swallow_exceptions`` is set."""
        n = len(trajectories)
        if n == 0:
            return []
        if n == 1:
            return [0.5]  # a relative score needs something to compare with
        body = {"model": self.cfg.judge_model, "messages": self.build_messages(trajectories), "temperature": 0.0, **self.cfg.sampling, **self.cfg.extra_body}
        err: Optional[BaseException] = None
        with self._lock:
            self.groups += 1
        for attempt in range(self.cfg.max_retries_on_parse_error + 1):
            try:
                reply = self.pool.chat(body)
                usage = reply.get("usage") or {}
                with self._lock:
                    self.input_tokens += int(usage.get("prompt_tokens") or 0)
                    self.output_tokens += int(usage.get("completion_tokens") or 0)
                return parse_scores(reply["choices"][0]["message"].get("content") or "", n)
            except (ValueError, KeyError, IndexError, TypeError) as e:   # a reply that does not parse: ask again
                err = e
                with self._lock:
                    self.parse_retries += 1
            except RulerJudgeError as e:
                err = e
                break
        with self._lock:
            self.failures += 1
        if self.cfg.swallow_exceptions:
            return None
        raise RulerJudgeError(f"the judge gave no usable scores for a group of {n}: {err}")

    # -- combination with the environment's reward
    def apply(self, trajectories: Sequence[Messages], rewards: Sequence[float]) -> Tuple[List[float], Dict[str, float]]:
        scores = self.score_group(trajectories)
        rewards = [float(r) for r in rewards]
        if scores is None:
            out = [0.0] * len(rewards) if self.cfg.mode == "replace" else rewards
            return out, {"ruler/failed": 1.0}
        w = self.cfg.weight
        if self.cfg.mode == "replace":
            out = [w * s for s in scores]
        elif self.cfg.mode == "add":
            out = [r + w * s for r, s in zip(rewards, scores)]
        else:
            out = rewards
        mean = sum(scores) / max(1, len(scores))
        return out, {"ruler/score_mean": mean, "ruler/score_spread": (max(scores) - min(scores)) if scores else 0.0, "ruler/failed": 0.0}

    def wrap_reward_fn(self, reward_fn: Optional[Callable[[Dict[str, Any], List[str]], List[float]]]):
        """A single-turn ``reward_fn(row, completions)`` with the judge applied on top (mode ``replace`` never calls the inner one)."""
        def fn(row: Dict[str, Any], completions: List[str]) -> List[float]:
            prompt = row.get("prompt")
            base = list(prompt) if isinstance(prompt, list) else [{"role": "user", "content": str(prompt)}]
            inner = [0.0] * len(completions) if (self.cfg.mode == "replace" or reward_fn is None) else reward_fn(row, completions)
            out, _ = self.apply([base + [{"role": "assistant", "content": c}] for c in completions], inner)
            return out

        return fn

    def metrics(self) -> Dict[str, float]:
        with self._lock:
            out = {"ruler/groups": float(self.groups), "ruler/failures": float(self.failures), "ruler/parse_retries": float(self.parse_retries),
                   "ruler/input_tokens": float(self.input_tokens), "ruler/output_tokens": float(self.output_tokens)}
            c = self.cfg.cost or {}
            if c.get("input_per_million") is not None or c.get("output_per_million") is not None:
                out["ruler/cost"] = (self.input_tokens * float(c.get("input_per_million") or 0.0) + self.output_tokens * float(c.get("output_per_million") or 0.0)) / 1e6
        return out


def build_ruler(raw: Optional[Dict[str, Any]], wait: bool = False, **pool_kw) -> Optional[RulerScorer]:
    cfg = RulerConfig.from_dict(raw)
    if not cfg.enabled:
        return None
    pool = JudgePool.from_config(cfg, **pool_kw)
    if wait:
        pool.wait_for_ready()
    return RulerScorer(cfg, pool)

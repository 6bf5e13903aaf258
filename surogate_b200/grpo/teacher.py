"""Teacher scores for rollouts: the log-probability a (larger) teacher model assigns to each sampled token.

The orchestrator asks an OpenAI-compatible server for ``prompt_logprobs`` of prompt + completion and keeps the completion part; the
trainer's ``ipo`` objective adds ``teacher_tau * (teacher log-prob - policy log-prob)`` to the advantage of every token, which pulls
the policy toward the teacher on its own samples (on-policy distillation) next to the task reward.

Parity: surogate/core/config/grpo_orch_config.py:56-80 (TeacherModelConfig), surogate/grpo/loss.py (teacher_tau).
"""
from __future__ import annotations

import itertools
import json
import os
import threading
import time
import urllib.request
from typing import Any, Dict, List, Optional, Sequence


class TeacherScorer:
    def __init__(self, base_urls: Sequence[str], model: str, api_key: str = "EMPTY", timeout_s: float = 600.0, max_retries: int = 3,
                 headers: Optional[Dict[str, str]] = None):
        self.urls = [u.rstrip("/") + "/completions" for u in base_urls]
        if not self.urls:
            raise ValueError("the teacher needs at least one base_url")
        self.model, self.key, self.timeout, self.max_retries, self.headers = model, api_key, timeout_s, max_retries, dict(headers or {})
        self._next, self._lock = itertools.cycle(range(len(self.urls))), threading.Lock()
        self.tokens_scored = 0

    @classmethod
    def from_config(cls, raw: Dict[str, Any]) -> Optional["TeacherScorer"]:
        """``{model: {name} | name, client: {base_url, api_key_var, timeout, headers}}`` or the flat ``{model, base_url, ...}``."""
        if not raw:
            return None
        model = raw.get("model")
        name = model.get("name") if isinstance(model, dict) else model
        client = raw.get("client") or raw
        urls = client.get("base_url") or client.get("base_urls")
        if not name or not urls:
            raise ValueError("teacher: give the model's name and the base_url of the server that serves it")
        urls = [urls] if isinstance(urls, str) else list(urls)
        var = client.get("api_key_var", "VLLM_API_KEY")
        return cls(urls, name, (os.environ.get(var) if var else None) or "EMPTY", float(client.get("timeout", 600.0)), headers=client.get("headers"))

    def logprobs(self, prompt_ids: Sequence[int], completion_ids: Sequence[int]) -> List[float]:
        """One log-prob per completion token (0.0 where the server returned none, which leaves that token's advantage as it is)."""
        ids = [int(t) for t in prompt_ids] + [int(t) for t in completion_ids]
        body = {"model": self.model, "prompt": ids, "max_tokens": 1, "temperature": 0.0, "prompt_logprobs": 1}
        last = None
        for attempt in range(self.max_retries + 1):
            with self._lock:
                url = self.urls[next(self._next)]
            req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json", "Authorization": f"Bearer {self.key}", **self.headers})
            try:
                with urllib.request.urlopen(req, timeout=self.timeout) as r:
                    entries = json.loads(r.read())["choices"][0].get("prompt_logprobs") or []
                break
            except Exception as e:  # noqa: BLE001 - retried alike
                last = e
                time.sleep(min(0.1 * 2.0 ** attempt, 5.0))
        else:
            raise RuntimeError(f"teacher at {self.urls} failed {self.max_retries + 1} times: {last}")
        out = []
        P = len(prompt_ids)
        for j, tok in enumerate(completion_ids):
            e = entries[P + j] if P + j < len(entries) else None
            v = (e or {}).get(str(int(tok)))
            out.append(float(v["logprob"] if isinstance(v, dict) else v) if v is not None else 0.0)
        with self._lock:
            self.tokens_scored += len(out)
        return out

    def score(self, rollouts) -> None:
        """Fill ``teacher_logprobs`` of every rollout (in place)."""
        for r in rollouts:
            r.teacher_logprobs = self.logprobs(r.prompt_ids, r.completion_ids)

"""Reward functions for the orchestrator: rule-based scorers and an LLM-judge group reward.

A reward function has the signature ``fn(prompt_row: dict, completions: list[str]) -> list[float]`` and scores the whole
group of completions of one prompt at once (which is what a relative judge needs).

Parity: surogate/rewards/ruler.py (LLM-judge group reward), environments/*.
"""
from __future__ import annotations

import importlib
import json
import re
import urllib.request
from typing import Callable, Dict, List

_NUM = re.compile(r"-?\d+(?:\.\d+)?")


def _final_answer(text: str) -> str:
    m = re.findall(r"\\boxed\{([^}]*)\}", text)
    if m:
        return m[-1].strip()
    m = re.findall(r"(?:answer|Answer)\s*(?:is|:)\s*([^\n]+)", text)
    if m:
        return m[-1].strip().rstrip(".")
    nums = _NUM.findall(text)
    return nums[-1] if nums else text.strip()


def exact_match(row: Dict, completions: List[str]) -> List[float]:
    gold = str(row.get("answer", "")).strip()
    return [1.0 if _final_answer(c) == gold else 0.0 for c in completions]


def length_penalised(row: Dict, completions: List[str]) -> List[float]:
    base = exact_match(row, completions)
    return [b - 1e-4 * len(c) for b, c in zip(base, completions)]


def format_reward(row: Dict, completions: List[str]) -> List[float]:
    """1 when the completion has a closed <think>...</think> block followed by an answer."""
    return [1.0 if re.search(r"<think>.*?</think>\s*\S", c, re.S) else 0.0 for c in completions]


class RulerJudge:
    """Relative LLM-judge reward: one request asks the judge model to score all completions of a prompt from 0 to 1."""

    def __init__(self, base_url: str, model: str, api_key: str = "EMPTY", timeout_s: float = 120.0, rubric: str = ""):
        self.url, self.model, self.key, self.timeout, self.rubric = base_url.rstrip("/") + "/chat/completions", model, api_key, timeout_s, rubric

    def __call__(self, row: Dict, completions: List[str]) -> List[float]:
        listing = "\n\n".join(f"<response id={i}>\n{c}\n</response>" for i, c in enumerate(completions))
        ask = (f"{self.rubric}\nTask given to the assistant:\n{row.get('prompt')}\n\nCandidate responses:\n{listing}\n\n"
               "Score every response between 0 and 1 relative to the others. Reply with JSON: {\"scores\": [..]} in id order.")
        body = json.dumps({"model": self.model, "messages": [{"role": "user", "content": ask}], "temperature": 0.0}).encode()
        req = urllib.request.Request(self.url, data=body, headers={"Content-Type": "application/json", "Authorization": f"Bearer {self.key}"})
        with urllib.request.urlopen(req, timeout=self.timeout) as r:
            text = json.loads(r.read())["choices"][0]["message"]["content"]
        m = re.search(r"\{.*\}", text, re.S)
        scores = json.loads(m.group(0))["scores"] if m else []
        if len(scores) != len(completions):
            return [0.0] * len(completions)
        return [min(1.0, max(0.0, float(s))) for s in scores]


REWARDS: Dict[str, Callable] = {"exact_match": exact_match, "length_penalised": length_penalised, "format": format_reward}


def resolve_reward(name: str) -> Callable:
    if name in REWARDS:
        return REWARDS[name]
    if ":" in name:
        mod, fn = name.split(":", 1)
        return getattr(importlib.import_module(mod), fn)
    raise ValueError(f"unknown reward '{name}' (known: {sorted(REWARDS)}, or module:function)")

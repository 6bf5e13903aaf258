"""A generic dataset-driven task scored by a judge model (relative ranking of a group of answers).

Rows come from a JSON-lines file; ``user_template`` is formatted with the row's fields to give the user message, the system
prompt is inline or read from a file.  Scoring has two modes: with ``judge_url`` the group of completions for one prompt is
ranked by an OpenAI-compatible judge (``grpo/rewards.py: RulerJudge``); without it (offline) the reward is exact match against
the row's ``answer_field``.

Parity: environments/ruler-task/ruler_task.py, surogate/rewards/ruler.py.
"""
from __future__ import annotations

import json
import string
from typing import Any, Dict, List, Optional

from .base import Rubric, SingleTurnEnv


def template_keys(template: str) -> List[str]:
    return [f for _, f, _, _ in string.Formatter().parse(template) if f]


def load_rows(path: str, max_examples: Optional[int] = None) -> List[Dict[str, Any]]:
    rows = []
    with open(path) as f:
        for line in f:
            if line.strip():
                rows.append(json.loads(line))
                if max_examples and len(rows) >= max_examples:
                    break
    return rows


def exact_match_reward(completion, answer, **_) -> float:
    text = completion if isinstance(completion, str) else completion[-1]["content"]
    return 1.0 if answer is not None and str(answer).strip().lower() in text.strip().lower() else 0.0


class RulerTaskEnv(SingleTurnEnv):
    env_id = "ruler-task"
    judge = None

    def score_group(self, example: Dict[str, Any], completions: List[str]) -> List[float]:
        """Relative scores for several completions of the same prompt (what group-relative policy optimisation consumes)."""
        if self.judge is not None:
            return self.judge({"prompt": example["prompt"], "answer": example.get("answer")}, completions)
        return [self.score(example, {"completion": c, "messages": [], "turns": 1})[0] for c in completions]


def load_environment(dataset_path: str = "", user_template: str = "{question}", answer_field: str = "answer", system_prompt: str = "",
                     system_prompt_path: Optional[str] = None, eval_path: Optional[str] = None, max_examples: Optional[int] = None,
                     judge_url: Optional[str] = None, judge_model: str = "", rubric: str = "", **_) -> RulerTaskEnv:
    if not dataset_path:
        raise ValueError("ruler-task needs dataset_path (a JSON-lines file)")
    if system_prompt_path:
        with open(system_prompt_path) as f:
            system_prompt = f.read()
    keys = template_keys(user_template)

    def to_example(row):
        missing = [k for k in keys if k not in row]
        if missing:
            raise KeyError(f"row lacks {missing} needed by the user template")
        return {"prompt": [{"role": "user", "content": user_template.format(**row)}], "answer": row.get(answer_field), "info": row}

    env = RulerTaskEnv([to_example(r) for r in load_rows(dataset_path, max_examples)], Rubric([exact_match_reward]),
                       [to_example(r) for r in load_rows(eval_path, max_examples)] if eval_path else None, system_prompt)
    if judge_url:
        from ..rewards import RulerJudge

        env.judge = RulerJudge(judge_url, judge_model, rubric=rubric)
    return env

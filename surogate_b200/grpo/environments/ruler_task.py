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


def _hub_rows(dataset: str, split: str, hf_config: Optional[str], limit: Optional[int]) -> List[Dict[str, Any]]:
    try:
        import datasets as hf_datasets  # type: ignore
    except ImportError as e:
        raise FileNotFoundError(f"dataset '{dataset}' is not a local file and the `datasets` package is not installed") from e
    ds = hf_datasets.load_dataset(dataset, hf_config, split=split)
    rows = [dict(r) for r in (ds.select(range(min(limit, len(ds)))) if limit else ds)]
    return rows


def load_environment(dataset_path: str = "", user_template: Optional[str] = None, answer_field: str = "answer", system_prompt: str = "",
                     system_prompt_path: Optional[str] = None, eval_path: Optional[str] = None, max_examples: Optional[int] = None,
                     judge_url: Optional[str] = None, judge_model: str = "", rubric: str = "", dataset: str = "", task_name: str = "", hf_config: Optional[str] = None,
                     dataset_split: str = "train", eval_split: Optional[str] = None, max_eval_examples: Optional[int] = None, seed: int = 42, shuffle: bool = False,
                     **other) -> RulerTaskEnv:
    """Rows -> single-turn prompts through ``user_template``; the reward is exact match where rows carry an answer, and otherwise
    comes from an LLM judge (``ruler`` section of the orchestrator config, or ``judge_url`` here).

    Two spellings of the source: ``dataset_path`` / ``eval_path`` (JSON-lines files, template default ``{question}``), or ``dataset``
    (a local file or a hub id with ``hf_config`` / ``dataset_split`` / ``eval_split``, template default ``{input}``) with
    ``task_name``, ``max_examples`` / ``max_eval_examples`` (None or -1 = all), ``seed`` / ``shuffle``."""
    unknown = sorted(k for k in other if k not in ("score_rollouts", "max_seq_len", "seq_len"))
    if unknown:
        raise ValueError(f"unrecognised arguments for ruler-task: {unknown}")
    limit = lambda n: None if n in (None, -1) else int(n)  # noqa: E731
    max_examples, max_eval_examples = limit(max_examples), limit(max_eval_examples)
    if user_template is None:
        user_template = "{input}" if dataset else "{question}"
    if not user_template.strip():
        raise ValueError("user_template must not be empty")
    if not dataset_path and not dataset:
        raise ValueError("ruler-task needs dataset_path (a JSON-lines file) or dataset (a file or a hub id)")
    if system_prompt_path:
        with open(system_prompt_path) as f:
            system_prompt = f.read()
    keys = template_keys(user_template)
    import os
    import random

    def rows_of(path_or_id: str, split: str, n: Optional[int]) -> List[Dict[str, Any]]:
        rows = load_rows(path_or_id, None if shuffle else n) if os.path.exists(path_or_id) else _hub_rows(path_or_id, split, hf_config, None if shuffle else n)
        if shuffle:
            random.Random(seed).shuffle(rows)
            rows = rows[:n] if n else rows
        return rows

    if dataset and not dataset_path:
        train_rows = rows_of(dataset, dataset_split, max_examples)
        eval_rows = rows_of(dataset, eval_split, max_eval_examples) if eval_split and not os.path.exists(dataset) else None

        def to_example_named(row):
            missing = [k for k in keys if k not in row]
            if missing:
                raise KeyError(f"row lacks {missing} needed by the user template")
            return {"prompt": [{"role": "user", "content": user_template.format(**row)}], "answer": row.get(answer_field), "info": dict(row, task_name=task_name),
                    "task": task_name or "ruler-task"}

        env = RulerTaskEnv([to_example_named(r) for r in train_rows], Rubric([exact_match_reward]), [to_example_named(r) for r in eval_rows] if eval_rows else None,
                           system_prompt)
        if judge_url:
            from ..rewards import RulerJudge

            env.judge = RulerJudge(judge_url, judge_model, rubric=rubric)
        return env

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

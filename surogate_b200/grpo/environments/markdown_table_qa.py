"""Markdown-table question answering (single turn).

The model gets a markdown table and a question, reasons inside ``<think>...</think>`` and gives the answer after the closing
tag.  One reward: correctness, checked by recomputing the answer from the table with pandas.  Numeric questions (sum, mean,
percentage, filtered sum / count) score 1 within 1 % (or 0.5 absolute) and fall off with the relative error; entity questions
(row with the max / min, top three) score by token F1 against the gold names.  Tables and questions are generated from a seed,
so the environment needs no download.

Parity: environments/markdown-table-qa/markdown_table_qa.py.
"""
from __future__ import annotations

import random
import re
from typing import Any, Dict, List, Optional

import pandas as pd

from .base import Rubric, SingleTurnEnv

MATH_TYPES = {"sum", "mean", "percentage", "filtered_sum", "filtered_count"}
ENTITY_TYPES = {"max_row", "min_row", "rank_top3"}
SYSTEM_PROMPT = ("You are a markdown table expert. Given a markdown table and a question, reason step by step inside <think>...</think> tags, "
                 "then give your final answer on a new line after the closing tag. Quote exact cell values, show arithmetic step by step, count only data "
                 "rows, and keep the final answer short and outside the think tags.")
NAMES = ["Avery", "Blake", "Casey", "Devon", "Emery", "Finley", "Gray", "Harper", "Indigo", "Jules", "Kai", "Logan", "Morgan", "Noel", "Oakley", "Parker"]
REGIONS = ["North", "South", "East", "West"]


def parse_markdown_table(md: str) -> Optional[pd.DataFrame]:
    lines = [l.strip() for l in md.strip().split("\n") if l.strip().startswith("|")]
    if len(lines) < 3:
        return None
    cols = [c.strip() for c in lines[0].split("|")[1:-1]]
    rows = [[c.strip() for c in l.split("|")[1:-1]] for l in lines[1:] if not re.match(r"^\|[\s\-:|]+\|$", l)]
    rows = [r for r in rows if len(r) == len(cols)]
    return pd.DataFrame(rows, columns=cols) if rows else None


def to_numeric(s: pd.Series) -> pd.Series:
    return pd.to_numeric(s.astype(str).str.replace(r"[,$%]", "", regex=True), errors="coerce")


def strip_think(text: str) -> str:
    text = re.sub(r"<think>.*?</think>", "", text, flags=re.S)
    return text.split("</think>")[-1].strip()


def final_number(text: str) -> Optional[float]:
    nums = re.findall(r"-?\d[\d,]*\.?\d*", strip_think(text))
    try:
        return float(nums[-1].replace(",", "")) if nums else None
    except ValueError:
        return None


def token_f1(pred: str, ref: str) -> float:
    p, r = re.findall(r"\w+", pred.lower()), re.findall(r"\w+", ref.lower())
    if not p or not r:
        return 0.0
    common = sum(min(p.count(t), r.count(t)) for t in set(r))
    if not common:
        return 0.0
    prec, rec = common / len(p), common / len(r)
    return 2 * prec * rec / (prec + rec)


def compute_gold(table_md: str, qtype: str, column: str, filter_value: Optional[str] = None) -> Dict[str, Any]:
    df = parse_markdown_table(table_md)
    if df is None or column not in df.columns:
        return {}
    vals = to_numeric(df[column])
    name_col = df.columns[0]
    if qtype == "sum":
        return {"value": float(vals.sum())}
    if qtype == "mean":
        return {"value": float(vals.mean())}
    if qtype in ("filtered_sum", "filtered_count", "percentage"):
        mask = df["Region"] == filter_value
        if qtype == "filtered_sum":
            return {"value": float(vals[mask].sum())}
        if qtype == "filtered_count":
            return {"value": float(mask.sum())}
        return {"value": float(100.0 * vals[mask].sum() / vals.sum())}
    if qtype == "max_row":
        return {"entity": str(df.loc[vals.idxmax(), name_col])}
    if qtype == "min_row":
        return {"entity": str(df.loc[vals.idxmin(), name_col])}
    if qtype == "rank_top3":
        return {"entity": ", ".join(df.loc[vals.sort_values(ascending=False).index[:3], name_col].astype(str))}
    return {}


def correctness_reward(completion, answer, info=None, **_) -> float:
    info = info or {}
    qtype = info.get("qtype", "")
    text = completion if isinstance(completion, str) else completion[-1]["content"]
    if qtype in MATH_TYPES:
        pred, gold = final_number(text), float(answer)
        if pred is None:
            return 0.0
        if abs(pred - gold) <= max(0.5, 0.01 * abs(gold)):
            return 1.0
        rel = abs(pred - gold) / max(abs(gold), 1e-9)
        return max(0.0, 0.5 * (1.0 - rel)) if rel < 1 else 0.0
    return token_f1(strip_think(text), str(answer))


def make_example(rng: random.Random) -> Dict[str, Any]:
    n = rng.randint(5, 9)
    names = rng.sample(NAMES, n)
    rows = [(nm, rng.choice(REGIONS), rng.randint(10, 500), rng.randint(1, 40)) for nm in names]
    while len({r[2] for r in rows}) < n:  # unique revenue keeps max / min / top-3 well defined
        rows = [(nm, reg, rng.randint(10, 500), u) for nm, reg, _, u in rows]
    md = "| Name | Region | Revenue | Units |\n|---|---|---|---|\n" + "\n".join(f"| {a} | {b} | {c} | {d} |" for a, b, c, d in rows)
    qtype = rng.choice(sorted(MATH_TYPES | ENTITY_TYPES))
    col = rng.choice(["Revenue", "Units"]) if qtype in ("sum", "mean") else "Revenue"
    region = rng.choice(sorted({r[1] for r in rows}))
    q = {"sum": f"What is the total {col}?", "mean": f"What is the average {col}?", "percentage": f"What percentage of total Revenue comes from the {region} region?",
         "filtered_sum": f"What is the total Revenue of the {region} region?", "filtered_count": f"How many rows are in the {region} region?",
         "max_row": "Who has the highest Revenue?", "min_row": "Who has the lowest Revenue?", "rank_top3": "List the top three names by Revenue, highest first."}[qtype]
    gold = compute_gold(md, qtype, col, region)
    answer = gold.get("value", gold.get("entity"))
    return {"prompt": [{"role": "user", "content": f"{md}\n\n{q}"}], "answer": answer, "info": {"qtype": qtype, "column": col, "region": region, "table": md}}


def load_environment(num_train: int = 512, num_eval: int = 64, seed: int = 0, max_examples: int = -1, **other) -> SingleTurnEnv:
    """Tables and questions are generated from the seed (nothing is downloaded), so ``hf_repo`` / ``split`` / ``focus_types`` of
    configs written for a hosted copy of the task are accepted without effect; ``max_examples`` > 0 is the other spelling of
    ``num_train``."""
    unknown = sorted(k for k in other if k not in ("hf_repo", "split", "focus_types", "score_rollouts", "max_seq_len", "seq_len"))
    if unknown:
        raise ValueError(f"unrecognised arguments for markdown-table-qa: {unknown}")
    if max_examples and int(max_examples) > 0:
        num_train = int(max_examples)
    rng = random.Random(seed)
    env = SingleTurnEnv([make_example(rng) for _ in range(num_train)], Rubric([correctness_reward]), [make_example(rng) for _ in range(num_eval)], SYSTEM_PROMPT)
    env.env_id = "markdown-table-qa"
    return env

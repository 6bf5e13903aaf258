"""Multi-hop question answering with a lookup tool (multi turn).

A seeded world of people linked in chains ("manager of", "mentor of", ...) with a few attributes each.  A question needs
``hops`` lookups ("What city does the manager of the mentor of X live in?").  The model calls the tool by writing
``<tool>{"name": "lookup", "args": {"entity": ..., "field": ...}}</tool>``; the environment answers in a ``tool`` message;
the episode ends when the model writes ``<answer>...</answer>`` (or runs out of turns).  Reward: 1 if the normalised answer
equals the gold one, else 0; a small bonus-free design keeps the signal unambiguous.

Parity: environments/multihop-tools/multihop_tools.py.
"""
from __future__ import annotations

import json
import random
import re
from typing import Any, Dict, List

from .base import Messages, MultiTurnEnv, Rubric

RELATIONS = ["manager", "mentor", "neighbor", "sibling"]
FIELDS = {"city": ["Oslo", "Lima", "Cairo", "Perth", "Quito", "Turin", "Hanoi", "Accra"], "pet": ["cat", "dog", "owl", "fox", "hen", "eel"],
          "color": ["red", "teal", "plum", "gold", "gray", "jade"]}
FIRST = ["Ada", "Ben", "Cy", "Dee", "Eli", "Fay", "Gus", "Hal", "Ivy", "Jon", "Kit", "Lou", "Max", "Nia", "Oz", "Pam", "Quin", "Rae", "Sol", "Tess"]
SYSTEM_PROMPT = ('Answer the question by looking facts up. To look something up write exactly <tool>{"name": "lookup", "args": {"entity": NAME, "field": FIELD}}</tool> '
                 "and wait for the result. Fields: " + ", ".join(RELATIONS + sorted(FIELDS)) + ". When you know the answer write <answer>ANSWER</answer>.")


def build_world(rng: random.Random, n_people: int = 16) -> Dict[str, Dict[str, Any]]:
    names = [f"{a} {b}son" for a, b in zip(rng.sample(FIRST, n_people), rng.sample(FIRST, n_people))]
    world = {}
    for nm in names:
        rec = {f: rng.choice(v) for f, v in FIELDS.items()}
        for rel in RELATIONS:
            rec[rel] = rng.choice([o for o in names if o != nm])
        world[nm] = rec
    return world


def make_question(world: Dict[str, Dict[str, Any]], rng: random.Random, hops: int):
    cur = rng.choice(sorted(world))
    start, rels = cur, []
    for _ in range(hops - 1):
        rel = rng.choice(RELATIONS)
        rels.append(rel)
        cur = world[cur][rel]
    field = rng.choice(sorted(FIELDS))
    phrase = start
    for rel in rels:
        phrase = f"the {rel} of {phrase}"
    return f"What is the {field} of {phrase}?", str(world[cur][field])


def norm(s: str) -> str:
    return re.sub(r"[^a-z0-9 ]", "", s.lower()).strip()


class MultiHopToolEnv(MultiTurnEnv):
    env_id = "multihop-tools"

    def setup_state(self, example):
        return {"world": example["info"]["world"], "tool_calls": 0}

    def is_completed(self, messages: Messages, state) -> bool:
        return "<answer>" in messages[-1]["content"]

    def env_response(self, messages: Messages, state) -> Messages:
        m = re.search(r"<tool>(.*?)</tool>", messages[-1]["content"], flags=re.S)
        if not m:
            return [{"role": "tool", "content": "error: no <tool> call and no <answer> found"}]
        state["tool_calls"] += 1
        try:
            call = json.loads(m.group(1))
            ent, field = call["args"]["entity"], call["args"]["field"]
            return [{"role": "tool", "content": str(state["world"][ent][field])}]
        except (ValueError, KeyError, TypeError) as e:
            return [{"role": "tool", "content": f"error: {type(e).__name__}"}]


def correctness_reward(completion, answer, **_) -> float:
    m = re.search(r"<answer>(.*?)</answer>", completion if isinstance(completion, str) else completion[-1]["content"], flags=re.S)
    return 1.0 if m and norm(m.group(1)) == norm(str(answer)) else 0.0


IGNORED_ARGS = ("score_rollouts", "max_seq_len", "seq_len", "n_chains")  # set by orchestrators of other layouts; nothing here depends on them


def load_environment(num_train: int = 256, num_eval: int = 32, hops: int = 3, max_turns: int = 8, seed: int = 0, num_examples: int = 0, min_hops: int = 0,
                     max_hops: int = 0, **other) -> MultiHopToolEnv:
    """``num_examples`` is the other spelling of ``num_train``; ``min_hops`` / ``max_hops`` draw the number of hops per question from
    a range instead of the fixed ``hops``."""
    unknown = sorted(k for k in other if k not in IGNORED_ARGS)
    if unknown:
        raise ValueError(f"unrecognised arguments for multihop-tools: {unknown}")
    rng = random.Random(seed)
    num_train = int(num_examples) or num_train
    lo, hi = (int(min_hops) or hops, int(max_hops) or hops) if (min_hops or max_hops) else (hops, hops)
    if lo > hi:
        raise ValueError(f"min_hops {lo} exceeds max_hops {hi}")

    def example():
        world = build_world(rng)
        n = rng.randint(lo, hi)
        q, a = make_question(world, rng, n)
        return {"prompt": [{"role": "user", "content": q}], "answer": a, "info": {"world": world, "hops": n}}

    return MultiHopToolEnv([example() for _ in range(num_train)], Rubric([correctness_reward]), [example() for _ in range(num_eval)], SYSTEM_PROMPT, max_turns=max_turns)

"""Example buffer with difficulty pools.

Every prompt ("example") lives in one of three pools.  After its group of rollouts is scored, a prompt whose mean reward is at
or above ``easy_threshold`` moves to *easy*, one at or below ``hard_threshold`` to *hard*, the rest stay *normal*.  Sampling
draws from *normal* only: prompts the policy always solves, or never solves, give all-equal rewards inside a group, hence
zero advantages and wasted generation.  When *normal* runs low a fraction of the other pools is recycled (the policy moves;
yesterday's hard prompt may be learnable today).  Scored rollouts wait in a rollout buffer until the trainer batch is drawn;
``online_difficulty_filtering`` drops groups with all-equal rewards before they get there.  State round-trips through jsonl
files, so a resumed orchestrator keeps its pools.

Parity: surogate/grpo/orchestrator/buffer.py:20-365.
"""
from __future__ import annotations

import hashlib
import json
import os
import random
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence

POOLS = ("easy", "normal", "hard")


@dataclass
class BufferConfig:
    seed: Optional[int] = 0
    easy_threshold: Optional[float] = None      # mean group reward >= this -> easy pool (None: never)
    hard_threshold: Optional[float] = None      # mean group reward <= this -> hard pool (None: never)
    easy_fraction: float = 0.25                 # share of the easy / hard pools returned to normal when it runs low
    hard_fraction: float = 0.25
    min_normal: int = 0                         # recycle when fewer examples than this remain in the normal pool
    online_difficulty_filtering: bool = True
    env_ratios: Optional[Sequence[float]] = None


class ExampleBuffer:
    def __init__(self, examples: Sequence[Dict[str, Any]], cfg: Optional[BufferConfig] = None, env_names: Optional[Sequence[str]] = None):
        self.cfg = cfg or BufferConfig()
        self.rng = random.Random(self.cfg.seed)
        if not examples:
            raise ValueError("the buffer needs at least one example")
        self.env_names = list(env_names) if env_names else sorted({e.get("task", "default") for e in examples})
        self.pools: Dict[str, Dict[str, Dict[int, Dict[str, Any]]]] = {p: {n: {} for n in self.env_names} for p in POOLS}
        seen = set()
        for i, e in enumerate(examples):
            e = dict(e)
            e.setdefault("example_id", i)
            e.setdefault("task", self.env_names[0])
            if e["example_id"] in seen:
                raise ValueError(f"duplicate example_id {e['example_id']}")
            seen.add(e["example_id"])
            if e["task"] not in self.pools["normal"]:
                raise ValueError(f"example {e['example_id']} names the unknown environment '{e['task']}'")
            self.pools["normal"][e["task"]][e["example_id"]] = e
        ratios = list(self.cfg.env_ratios) if self.cfg.env_ratios else [len(self.pools["normal"][n]) for n in self.env_names]
        total = float(sum(ratios)) or 1.0
        self.env_probs = {n: r / total for n, r in zip(self.env_names, ratios)}
        self.rollouts: List[Any] = []
        self.reset_step_metrics()

    # ------------------------------------------------------------------ bookkeeping
    @staticmethod
    def example_hash(example: Dict[str, Any]) -> str:
        return hashlib.sha256(json.dumps({"task": example.get("task"), "prompt": example.get("prompt")}, sort_keys=True, default=str).encode()).hexdigest()

    def count(self, pool: str) -> int:
        return sum(len(v) for v in self.pools[pool].values())

    def reset_step_metrics(self) -> None:
        self.step = {"to_easy": 0, "to_hard": 0, "filtered_groups": 0, "groups": 0, "recycled": 0}

    def _recycle_if_needed(self) -> None:
        if self.count("normal") > self.cfg.min_normal:
            return
        for pool, frac in (("easy", self.cfg.easy_fraction), ("hard", self.cfg.hard_fraction)):
            for env in self.env_names:
                ids = list(self.pools[pool][env])
                take = ids if self.count("normal") == 0 and frac <= 0 else self.rng.sample(ids, int(round(len(ids) * frac))) if ids else []
                for i in take:
                    self.pools["normal"][env][i] = self.pools[pool][env].pop(i)
                    self.step["recycled"] += 1
        if self.count("normal") == 0:   # everything is classified and the fractions are zero: start over rather than stall
            for pool in ("easy", "hard"):
                for env in self.env_names:
                    self.pools["normal"][env].update(self.pools[pool][env])
                    self.pools[pool][env].clear()

    # ------------------------------------------------------------------ prompts out
    def sample_examples(self, n: int) -> List[Dict[str, Any]]:
        self._recycle_if_needed()
        out = []
        envs = [e for e in self.env_names if self.pools["normal"][e]]
        for _ in range(n):
            if not envs:
                break
            env = self.rng.choices(envs, weights=[self.env_probs[e] for e in envs])[0]
            ex = self.rng.choice(list(self.pools["normal"][env].values()))
            out.append(ex)
        return out

    # ------------------------------------------------------------------ scored rollouts in
    def update(self, groups: Sequence[Sequence[Any]]) -> None:
        """``groups``: per prompt, its scored rollouts (objects with ``reward`` and ``meta['example_id' / 'task']``)."""
        for g in groups:
            if not g:
                continue
            self.step["groups"] += 1
            rewards = [float(r.reward) for r in g]
            mean = sum(rewards) / len(rewards)
            ex_id, task = g[0].meta.get("example_id"), g[0].meta.get("task", self.env_names[0])
            src = next((p for p in POOLS if ex_id in self.pools[p].get(task, {})), None)
            dst = "normal"
            if self.cfg.easy_threshold is not None and mean >= self.cfg.easy_threshold:
                dst = "easy"
            elif self.cfg.hard_threshold is not None and mean <= self.cfg.hard_threshold:
                dst = "hard"
            if src is not None and src != dst:
                self.pools[dst][task][ex_id] = self.pools[src][task].pop(ex_id)
                self.step["to_" + dst] += dst != "normal"
            if self.cfg.online_difficulty_filtering and max(rewards) == min(rewards):
                self.step["filtered_groups"] += 1
                continue
            self.rollouts.extend(g)

    def sample_rollouts(self, n: int) -> List[Any]:
        """The oldest ``n`` buffered rollouts (all of a step's batch comes from here, in arrival order)."""
        out, self.rollouts = self.rollouts[:n], self.rollouts[n:]
        return out

    def metrics(self) -> Dict[str, float]:
        total = max(1, sum(self.count(p) for p in POOLS))
        m = {f"buffer/{p}": self.count(p) / total for p in POOLS}
        m.update({f"buffer/{k}": float(v) for k, v in self.step.items()})
        m["buffer/pending_rollouts"] = float(len(self.rollouts))
        return m

    # ------------------------------------------------------------------ persistence
    def save(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        for p in POOLS:
            with open(os.path.join(path, f"{p}_examples.jsonl"), "w") as f:
                for env in self.env_names:
                    for ex in self.pools[p][env].values():
                        f.write(json.dumps({"hash": self.example_hash(ex), "example_id": ex["example_id"], "task": ex["task"]}) + "\n")

    def load(self, path: str) -> int:
        """Re-applies saved pool membership by example hash (the dataset may have been re-ordered or extended); returns how many
        examples were moved."""
        by_hash = {self.example_hash(ex): (p, env, i) for p in POOLS for env in self.env_names for i, ex in self.pools[p][env].items()}
        moved = 0
        for p in ("easy", "hard"):
            fn = os.path.join(path, f"{p}_examples.jsonl")
            if not os.path.exists(fn):
                continue
            with open(fn) as f:
                for line in f:
                    rec = json.loads(line)
                    at = by_hash.get(rec["hash"])
                    if at is None or at[0] == p:
                        continue
                    src, env, i = at
                    self.pools[p][env][i] = self.pools[src][env].pop(i)
                    by_hash[rec["hash"]] = (p, env, i)
                    moved += 1
        return moved

"""``surogate vf-init <env-id>`` scaffolds an environment package; ``surogate vf-eval <env-id>`` evaluates a model on one.

Parity: surogate/cli/vf_init.py, surogate/cli/vf_eval.py.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

README = """# {dash}

### Overview
- **Environment ID**: `{dash}`
- **Short description**: <one sentence>

### Task
- **Type**: <single-turn | multi-turn | tool use>
- **Rubric**: <reward functions and weights>

### Quickstart
```bash
surogate vf-eval -m <model> -b http://127.0.0.1:8000/v1 -n 20 -r 3 -a '{{"key": "value"}}' {dash}
```
"""

MODULE = '''"""{dash}: describe the task here."""
from surogate_b200.grpo.environments import Rubric, SingleTurnEnv


def correctness_reward(completion, answer, **_):
    return 1.0 if str(answer).strip() in completion else 0.0


def load_environment(**kwargs):
    data = [{{"prompt": [{{"role": "user", "content": "What is 2 + 2?"}}], "answer": "4"}}]
    env = SingleTurnEnv(data, Rubric([correctness_reward]), data, system_prompt="Answer briefly.")
    env.env_id = "{dash}"
    return env
'''

PYPROJECT = """[project]
name = "{dash}"
version = "0.1.0"
description = "RL environment {dash}"
dependencies = []
"""


def init_environment(env_id: str, path: str = "./environments") -> str:
    dash, under = env_id.replace("_", "-"), env_id.replace("-", "_")
    root = os.path.join(path, under)
    os.makedirs(root, exist_ok=True)
    for name, text in (("README.md", README), (under + ".py", MODULE), ("pyproject.toml", PYPROJECT)):
        target = os.path.join(root, name)
        if not os.path.exists(target):
            with open(target, "w") as f:
                f.write(text.format(dash=dash))
    return root


def main(argv, command: str = "vf-eval") -> int:
    if command == "vf-init":
        p = argparse.ArgumentParser(prog="surogate vf-init")
        p.add_argument("env")
        p.add_argument("--path", "-p", default="./environments")
        a = p.parse_args(argv)
        print(init_environment(a.env, a.path))
        return 0
    p = argparse.ArgumentParser(prog="surogate vf-eval")
    p.add_argument("env", help="environment id (built in, scaffolded under the environments directory, or importable with --env-path)")
    p.add_argument("--env-args", "-a", default="{}", help="environment arguments as a JSON object")
    p.add_argument("--env-dir-path", "--path", "-p", dest="path", default="./environments", help="environments directory")
    p.add_argument("--env-path", default=None, help="directory put in front of sys.path before importing the environment's package")
    p.add_argument("--model", "-m", default="")
    p.add_argument("--api-base-url", "--base-url", "-b", dest="base_url", default="http://127.0.0.1:8000/v1")
    p.add_argument("--api-key-var", "-k", default=None, help="environment variable with the API key (EMPTY when unset)")
    p.add_argument("--header", action="append", default=None, help="extra HTTP header 'Name: Value' (repeatable)")
    p.add_argument("--num-examples", "-n", type=int, default=20)
    p.add_argument("--rollouts-per-example", "-r", type=int, default=1)
    p.add_argument("--max-concurrent", "-c", type=int, default=32, help="rollouts in flight")
    p.add_argument("--max-tokens", "-t", type=int, default=1024)
    p.add_argument("--temperature", "-T", type=float, default=0.7)
    p.add_argument("--sampling-args", "-S", default="{}", help="extra sampling arguments merged into every request, as a JSON object")
    p.add_argument("--max-retries", type=int, default=0)
    p.add_argument("--verbose", "-v", action="store_true", help="print every sample's reward as it is scored")
    p.add_argument("--save-results", "--save", "-s", dest="save", default=None, help="write the full result (with samples) to this JSON file")
    a = p.parse_args(argv)
    from ..grpo.environments import evaluate, load_environment, openai_policy

    headers = {}
    for h in a.header or []:
        name, sep, value = h.partition(":")
        if not sep or not name.strip():
            p.error(f"--header must be 'Name: Value', got {h!r}")
        headers[name.strip()] = value.strip()
    key = (os.environ.get(a.api_key_var) if a.api_key_var else None) or "EMPTY"
    env = load_environment(a.env, path=a.path, import_path=a.env_path, **json.loads(a.env_args))
    policy = openai_policy(a.base_url, a.model, a.temperature, a.max_tokens, api_key=key, headers=headers, sampling_args=json.loads(a.sampling_args),
                           max_retries=a.max_retries)
    on_sample = (lambda s: print(f"reward {s['reward']:.3f}  turns {s['turns']}", file=sys.stderr)) if a.verbose else None
    res = evaluate(env, policy, a.num_examples, a.rollouts_per_example, max_concurrent=a.max_concurrent, on_sample=on_sample)
    if a.save:
        with open(a.save, "w") as f:
            json.dump(res, f, indent=1)
    print(json.dumps({k: v for k, v in res.items() if k != "samples"}))
    return 0

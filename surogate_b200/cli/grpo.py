"""The GRPO commands.

    surogate grpo          --train T.yaml --infer I.yaml --orch O.yaml --trainer-gpus 0,1 --vllm-gpus 2,3 [--judge-infer J.yaml --judge-gpus 4]
    surogate grpo-colocate --train T.yaml --infer I.yaml --orch O.yaml [--gpus 0,1]
    surogate grpo-train  T.yaml      surogate grpo-orch  O.yaml      surogate grpo-infer  I.yaml

``grpo`` runs trainer, rollout engine and orchestrator on disjoint GPU sets under one supervisor, ``grpo-colocate`` on shared
GPUs; ``grpo-train`` is the trainer alone (consumes rollout batches, publishes weights), ``grpo-orch`` the orchestrator (prompts
-> rollouts -> rewards -> batches), ``grpo-infer`` launches the rollout engine and keeps it on the newest published weights.
``grpo`` and ``grpo-train`` are told apart by their arguments, so either name works for either form: with ``--train`` it is
the supervised three-component run, with one positional config it is the trainer.  ``--trainer-gpus 0,1`` on the trainer pins
its devices before CUDA is initialised (handled in cli/main.py).

Parity: surogate/cli/{grpo,grpo_colocate,grpo_train,grpo_orch,grpo_infer}.py, surogate/grpo/{trainer,split,colocate}.py.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def is_supervised(argv) -> bool:
    """True for the three-component form (``--train T.yaml ...``), False for the trainer's ``config.yaml`` form."""
    return any(a == "--train" or a.startswith("--train=") for a in argv)


def _run_all(argv, command: str) -> int:
    """``grpo --train T.yaml --infer I.yaml --orch O.yaml --trainer-gpus 0-3 --vllm-gpus 4-7`` (disjoint GPU sets) and
    ``grpo-colocate --train T.yaml --infer I.yaml --orch O.yaml [--gpus 0-7]`` (shared GPUs): one supervisor, three components."""
    split = command != "grpo-colocate"
    from ..grpo.runners import Supervisor, plan_colocate, plan_split

    p = argparse.ArgumentParser(prog=f"surogate {command}")
    p.add_argument("--train", required=True)
    p.add_argument("--infer", required=True)
    p.add_argument("--orch", required=True)
    p.add_argument("--max-steps", type=int, default=None, dest="max_steps")
    p.add_argument("--dry-run", action="store_true", help="print the component commands and exit")
    if split:
        p.add_argument("--trainer-gpus", required=True)
        p.add_argument("--vllm-gpus", required=True)
        p.add_argument("--judge-infer", "--judge-config", dest="judge_config", default=None, help="inference config of a judge engine started next to the rollout engine")
        p.add_argument("--judge-gpus", default=None)
    else:
        p.add_argument("--gpus", default=None)
        p.add_argument("--engine-memory-fraction", type=float, default=None)
    a = p.parse_args(argv)
    from ..config.loader import read_yaml

    raw = read_yaml(a.infer)
    tp, dp = int(raw.get("tp") or raw.get("tensor_parallel_size", 1)), int(raw.get("dp") or raw.get("data_parallel_size", 1))
    if split:
        jraw = read_yaml(a.judge_config) if a.judge_config else {}
        jtp = int(jraw.get("tp") or jraw.get("tensor_parallel_size", 1))
        comps = plan_split(a.train, a.infer, a.orch, a.trainer_gpus, a.vllm_gpus, tp, dp, a.judge_config, a.judge_gpus, jtp, max_steps=a.max_steps)
    else:
        comps = plan_colocate(a.train, a.infer, a.orch, a.gpus, max_steps=a.max_steps,
                              engine_memory_fraction=a.engine_memory_fraction or float(raw.get("gpu_memory_utilization", 0.45)))
    if a.dry_run:
        for c in comps:
            print(json.dumps({"name": c.name, "argv": c.argv, "env": c.env}))
        return 0
    return Supervisor(comps, reap=True).run()


def main(argv, command: str = "grpo") -> int:
    if command == "grpo-colocate" or (command in ("grpo", "grpo-train") and is_supervised(argv)):
        return _run_all(argv, command)
    if command == "grpo-train":
        command = "grpo"
    p = argparse.ArgumentParser(prog=f"surogate {command}")
    p.add_argument("config")
    p.add_argument("--trainer-gpus", default=None)
    p.add_argument("--max-steps", type=int, default=None, dest="max_steps")
    a = p.parse_args(argv)
    from ..config.loader import load_config, read_yaml

    if command == "grpo":
        from ..grpo.config import GRPOConfig
        from ..grpo.trainer import run_grpo

        r = run_grpo(load_config(GRPOConfig, a.config, max_steps=a.max_steps))
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"steps": r["steps"], "final": r["history"][-1] if r["history"] else None}))
        return 0
    raw = read_yaml(a.config)
    if command == "grpo-orch":
        from ..grpo.config_compat import flatten_orchestrator_config

        raw, notes = flatten_orchestrator_config(raw)   # a config in the nested orchestrator schema becomes this package's flat keys
        for n in notes:
            print(f"[grpo-orch] {n}", file=sys.stderr)
        from ..data.tokenizer import Tokenizer
        from ..grpo.config import OrchestratorConfig
        from ..grpo.orchestrator import OpenAIClient, Orchestrator
        from ..grpo.transport import make_transport
        from ..grpo.weight_broadcast import FilesystemBroadcast

        from ..config.loader import coerce_fields

        cfg = OrchestratorConfig(**coerce_fields(OrchestratorConfig, {k: v for k, v in raw.items() if k in OrchestratorConfig.__dataclass_fields__}))
        if a.max_steps:
            cfg.max_steps = a.max_steps
        b = FilesystemBroadcast(cfg.weight_dir)
        served = raw.get("served_model") or cfg.model            # the name requests carry (an adapter registered with the engine, or the model)
        key = (os.environ.get(raw["api_key_var"]) if raw.get("api_key_var") else None) or "EMPTY"
        headers = raw.get("headers") or {}

        def client(url):
            return OpenAIClient(url, served, cfg.request_timeout_s, api_key=key, headers=headers)

        orch = Orchestrator(cfg, Tokenizer.from_pretrained(cfg.model), client(cfg.base_url),
                            make_transport(cfg.transport, directory=cfg.transport_dir, endpoint=cfg.zmq_endpoint, role="producer"),
                            lambda: (b.latest() or {"version": -1})["version"])
        if orch.judge is not None:
            orch.judge.pool.wait_for_ready()   # a judge engine started next to this run needs a while to load
        orch.load_prompts()
        if raw.get("async_scheduler") or raw.get("scheduler") == "async":
            # asynchronous loop: bounded in-flight requests on a thread pool, difficulty pools, rollout filters, depth budget
            from ..grpo.orchestration import AsyncOrchestrator, async_config_from, make_generate_group

            urls = raw.get("base_urls") or [cfg.base_url]
            if len(urls) > 1:
                orch.client = [client(u) for u in urls]
            tok = orch.tok
            acfg = async_config_from(cfg, raw, vocab_size=getattr(tok, "vocab_size", 32000), pad_token_id=max(0, getattr(tok, "pad_token_id", 0)))
            eval_rows = None
            if acfg.eval_every and raw.get("eval_environments"):
                eval_rows = orch.add_eval_environments(raw["eval_environments"], raw.get("eval_examples"))
            elif acfg.eval_every and orch.env is not None and getattr(orch.env, "eval_dataset", None):
                eval_rows = [dict(ex, prompt=orch.env.initial_messages(ex)) for ex in orch.env.eval_dataset][:raw.get("eval_examples") or None]
            loop = AsyncOrchestrator(acfg, orch.prompts, make_generate_group(orch), orch.transport, lambda: (b.latest() or {"version": -1})["version"],
                                     num_servers=len(urls), eval_examples=eval_rows, env_names=list(orch.envs) or None)
            hist = loop.run()
            print(json.dumps({"steps": len(hist), "last_reward_mean": hist[-1].get("reward/mean") if hist else None}))
            return 0
        hist = orch.run()
        print(json.dumps({"steps": len(hist), "last_reward_mean": hist[-1].reward_mean if hist else None}))
        return 0
    from ..grpo.config import InferenceConfig
    from ..grpo.inference import launch_server, watch_and_reload

    from ..config.loader import coerce_fields

    unknown = sorted(k for k in raw if k not in InferenceConfig.__dataclass_fields__)
    if unknown:
        print(f"[grpo-infer] keys without effect: {', '.join(unknown)}", file=sys.stderr)
    cfg = InferenceConfig(**coerce_fields(InferenceConfig, {k: v for k, v in raw.items() if k in InferenceConfig.__dataclass_fields__}))
    proc = launch_server(cfg)
    try:
        watch_and_reload(cfg, f"http://{cfg.host}:{cfg.port}/v1")
    finally:
        proc.terminate()
    return 0

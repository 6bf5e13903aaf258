"""Run small training cases and compare them with stored baselines.

A case fixes model shape, recipe, optimizer, sharding level, offload mode and seeds, trains a few steps on synthetic
tokens and records: the loss curve, gradient norms, step-time p50 / p95, peak device memory and a summary of the
parameter-store layout (bucket count, bytes per category).  ``compare`` checks a fresh artifact against a baseline with
tolerances per field; the CLI entry (``python -m surogate_b200.regression.runner``) runs the matrix and writes
``regression_baselines/<case>.json`` or reports differences.

Parity: surogate/regression/baseline_runner.py, regression_baselines/.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import statistics
import sys
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import numpy as np


@dataclass
class Case:
    name: str
    model: Dict[str, Any]
    recipe: str = "bf16"
    optimizer: str = "adamw_8bit"
    zero_level: int = 0
    lora: Optional[Dict[str, Any]] = None
    offload: str = "none"  # none | offload | cpu_training
    recompute: bool = False
    batch: int = 2
    seq_len: int = 64
    steps: int = 6
    lr: float = 1e-3
    seed: int = 0
    needs_gpu: bool = False


TINY = dict(architecture="Qwen3ForCausalLM", vocab_size=512, d_model=128, n_layers=2, num_query_heads=4, num_kv_heads=2, head_size=32, d_ff=256,
            tie_word_embeddings=True)
TINY_GPU = dict(TINY, head_size=128, d_model=512, d_ff=1024)
TINY_MOE = dict(architecture="Qwen3MoeForCausalLM", vocab_size=512, d_model=128, n_layers=2, num_query_heads=4, num_kv_heads=2, head_size=32, moe_d_ff=64,
                num_experts=8, num_experts_per_tok=2, aux_loss_coef=1e-2, tie_word_embeddings=False)
LORA = dict(rank=8, alpha=16, dropout=0.0, dtype="fp32", targets=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"], rslora=False,
            train_router=False)


def default_matrix(gpu: bool) -> List[Case]:
    cases = [Case("dense-bf16-adamw", TINY, optimizer="adamw"), Case("dense-bf16-adamw8", TINY), Case("dense-bf16-recompute", TINY, recompute=True),
             Case("dense-lora", TINY, lora=LORA, optimizer="adamw"), Case("dense-offload", TINY, offload="offload", optimizer="adamw"),
             Case("dense-cpu-training", TINY, offload="cpu_training", optimizer="adamw"), Case("moe-bf16", TINY_MOE, optimizer="adamw")]
    if gpu:
        cases += [Case("gpu-dense-fp8", TINY_GPU, recipe="fp8_hybrid", seq_len=256, needs_gpu=True),
                  Case("gpu-dense-nvfp4", TINY_GPU, recipe="nvfp4", seq_len=256, needs_gpu=True),
                  Case("gpu-dense-normuon", TINY_GPU, optimizer="normuon", seq_len=256, needs_gpu=True)]
    return cases


def run_case(case: Case, device: Optional[str] = None) -> Dict[str, Any]:
    import torch

    from ..runtime.trainer import Trainer, TrainerConfig

    dev = torch.device(device or ("cuda" if (torch.cuda.is_available() and case.needs_gpu) else "cpu"))
    kw = {"offload": dict(offload_master=True, offload_optimizer=True), "cpu_training": dict(cpu_training=True)}.get(case.offload, {})
    cfg = TrainerConfig(model=case.model, batch_size=case.batch, seq_len=case.seq_len, recipe=case.recipe, optimizer=case.optimizer, learning_rate=case.lr,
                        zero_level=case.zero_level, recompute=case.recompute, lora=case.lora, seed=case.seed, **kw)
    tr = Trainer(cfg, device=dev)
    tr.init_weights(case.seed)
    rng = np.random.default_rng(case.seed + 1)
    V = case.model["vocab_size"]
    tok = rng.integers(0, V, (case.batch, case.seq_len + 1)).astype(np.int32)
    losses, norms, times = [], [], []
    if dev.type == "cuda":
        torch.cuda.reset_peak_memory_stats(dev)
    for _ in range(case.steps):
        t0 = time.perf_counter()
        out = tr.step(tok[:, :-1], tok[:, 1:])
        times.append((time.perf_counter() - t0) * 1e3)
        losses.append(out["loss"])
        norms.append(out["norm"])
    mem = tr.memory_breakdown()
    ts = sorted(times[1:] or times)
    try:   # the graph compiler's static buffer plan: a changed fusion rule or liveness analysis shows up here before it shows in memory
        plan = tr.activation_plan()
        plan_summary = {"saved_bytes": int(plan.saved_bytes), "temp_bytes": int(plan.temp_bytes),
                        "tensors": {bt: {ph: len(p.tensors) for ph, p in phases.items()} for bt, phases in plan.per_block.items()}}
    except Exception:  # noqa: BLE001 - a model whose graphs the planner does not cover: the artifact goes without
        plan_summary = None
    return {"case": dataclasses.asdict(case), "device": dev.type, "losses": losses, "norms": norms, "plan": plan_summary,
            "step_ms_p50": statistics.median(ts), "step_ms_p95": ts[min(len(ts) - 1, int(0.95 * len(ts)))],
            "peak_memory": mem.get("peak", 0), "store": {"buckets": len(tr.store.buckets), **{k: v for k, v in mem.items() if k in ("master", "work", "grad", "host_master")}},
            "num_parameters": tr.num_parameters()}


def compare(new: Dict[str, Any], base: Dict[str, Any], loss_rtol: float = 2e-2, time_factor: float = 1.5, mem_factor: float = 1.15) -> List[str]:
    problems = []
    if len(new["losses"]) != len(base["losses"]):
        problems.append(f"step count {len(new['losses'])} != {len(base['losses'])}")
    for i, (a, b) in enumerate(zip(new["losses"], base["losses"])):
        if abs(a - b) > loss_rtol * max(abs(b), 1e-6):
            problems.append(f"loss[{i}] {a:.5f} vs baseline {b:.5f}")
            break
    if new["device"] == base["device"] and new["step_ms_p50"] > time_factor * base["step_ms_p50"]:
        problems.append(f"step time p50 {new['step_ms_p50']:.1f} ms > {time_factor}x baseline {base['step_ms_p50']:.1f} ms")
    if base.get("peak_memory") and new.get("peak_memory", 0) > mem_factor * base["peak_memory"]:
        problems.append(f"peak memory {new['peak_memory']} > {mem_factor}x baseline {base['peak_memory']}")
    if new["store"]["buckets"] != base["store"]["buckets"] or new["num_parameters"] != base["num_parameters"]:
        problems.append("parameter-store layout changed")
    if base.get("plan") and new.get("plan") and (new["plan"]["saved_bytes"] != base["plan"]["saved_bytes"] or new["plan"]["tensors"] != base["plan"]["tensors"]):
        problems.append(f"buffer plan changed: saved bytes {new['plan']['saved_bytes']} vs {base['plan']['saved_bytes']}, tensors {new['plan']['tensors']} vs {base['plan']['tensors']}")
    return problems


DEFAULT_RUN_TIMEOUT_S = int(os.environ.get("SUROGATE_REGRESSION_TIMEOUT_S", "1800"))


def run_config(config_path: str, artifact_path: str, command: str = "sft", timeout_s: Optional[int] = None, extra_env: Optional[Dict[str, str]] = None) -> Dict[str, Any]:
    """One real training config as a subprocess (``surogate <command> <config>``) that writes its artifact where
    ``SUROGATE_REGRESSION_ARTIFACT`` points; returns the artifact.  A run that fails or outlasts ``timeout_s``
    (``SUROGATE_REGRESSION_TIMEOUT_S``, default 1800) raises with the end of its output.
    Parity: surogate/regression/baseline_runner.py:300-330."""
    import subprocess

    env = dict(os.environ, SUROGATE_REGRESSION_ARTIFACT=artifact_path, SUROGATE_NO_BANNER="1", **(extra_env or {}))
    if os.path.exists(artifact_path):
        os.remove(artifact_path)
    try:
        r = subprocess.run([sys.executable, "-m", "surogate_b200.cli.main", command, config_path], env=env, capture_output=True, text=True,
                           timeout=timeout_s or DEFAULT_RUN_TIMEOUT_S)
    except subprocess.TimeoutExpired as e:
        raise RuntimeError(f"{config_path}: no result after {e.timeout:.0f} s") from e
    if r.returncode != 0 or not os.path.exists(artifact_path):
        raise RuntimeError(f"{config_path}: exit code {r.returncode}, artifact {'missing' if not os.path.exists(artifact_path) else 'present'}\n{(r.stdout + r.stderr)[-2000:]}")
    with open(artifact_path) as f:
        return json.load(f)


def run_configs(paths: List[str], baselines: str, update: bool) -> int:
    """Each config as a subprocess; baseline ``<baselines>/<config file name>.json`` written (first run / ``update``) or compared."""
    from .artifact import compare_runs

    failed = 0
    for cfg in paths:
        name = os.path.splitext(os.path.basename(cfg))[0]
        base = os.path.join(baselines, name + ".json")
        new = os.path.join(baselines, name + ".new.json")
        try:
            art = run_config(cfg, new)
        except RuntimeError as e:
            print(f"[FAIL] {name}: {e}")
            failed += 1
            continue
        if update or not os.path.exists(base):
            os.replace(new, base)
            print(f"[baseline] {name}: wrote {base}")
            continue
        with open(base) as f:
            problems = compare_runs(art, json.load(f))
        os.remove(new)
        print(f"[{'FAIL' if problems else ' ok '}] {name}" + ("".join("\n    " + x for x in problems)))
        failed += bool(problems)
    return failed


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m surogate_b200.regression.runner")
    p.add_argument("--baselines", default="regression_baselines")
    p.add_argument("--update", action="store_true", help="write / overwrite baselines instead of comparing")
    p.add_argument("--only", default=None)
    p.add_argument("--config", action="append", default=[], help="a training config to run as a subprocess and compare (repeatable); without it the built-in matrix runs")
    a = p.parse_args(argv)
    import torch

    os.makedirs(a.baselines, exist_ok=True)
    if a.config:
        return 1 if run_configs(a.config, a.baselines, a.update) else 0
    failed = 0
    for case in default_matrix(torch.cuda.is_available()):
        if a.only and a.only not in case.name:
            continue
        art = run_case(case)
        path = os.path.join(a.baselines, case.name + ".json")
        if a.update or not os.path.exists(path):
            with open(path, "w") as f:
                json.dump(art, f, indent=1)
            print(f"[baseline] {case.name}: wrote {path}")
            continue
        with open(path) as f:
            problems = compare(art, json.load(f))
        print(f"[{'FAIL' if problems else ' ok '}] {case.name}" + ("".join("\n    " + x for x in problems)))
        failed += bool(problems)
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())

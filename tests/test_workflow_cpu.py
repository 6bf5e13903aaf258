"""Workflow helpers on CPU: stage planner, multi-node launch plan, reporters, plots, regression harness, SFT with adapters."""
import json
import os
import sys

import numpy as np
import pytest

from surogate_b200.train.dispatch_pp import plan_stages, wavefront


def test_dispatch_pp_plan_and_wavefront():
    st = plan_stages(36, 4, stage_layers=4)
    assert len(st) == 9 and [s.gpu for s in st[:5]] == [0, 1, 2, 3, 0]
    assert st[0].first_layer == 0 and st[-1].last_layer == 36 and all(a.last_layer == b.first_layer for a, b in zip(st, st[1:]))
    assert len(plan_stages(2, 4)) == 2  # never more stages than layers
    ticks = wavefront(3, 4)
    fwd = [t for t in ticks if t and t[0][0] == "fwd"]
    assert len(fwd) == 6 and fwd[0] == [("fwd", 0, 0)] and set(fwd[2]) == {("fwd", 0, 2), ("fwd", 1, 1), ("fwd", 2, 0)}
    seen = {(p, s, m) for t in ticks for p, s, m in t}
    assert len(seen) == 2 * 3 * 4
    order = {(p, s, m): i for i, t in enumerate(ticks) for p, s, m in t}
    for m in range(4):  # dependencies: stage s after stage s-1 (forward), stage s after stage s+1 (backward), backward after forward
        assert order[("fwd", 1, m)] > order[("fwd", 0, m)] and order[("bwd", 0, m)] > order[("bwd", 1, m)] > order[("fwd", 2, m)]


def test_multinode_plan_and_interface_detection(monkeypatch):
    from surogate_b200.train import distributed as d

    plan = d.plan_launch("cfg.yaml", "sft", 2, 8, "10.0.0.1", 29500)
    assert len(plan) == 2 and "--node-rank=1" in plan[1].command and "--nproc-per-node=8" in plan[0].command
    assert plan[0].command[-3:] == ["surogate_b200.cli.main", "sft", "cfg.yaml"][-3:]
    cmds = d.launch_over_ssh(["a", "b"], "cfg.yaml", "pt", 8, dry_run=True)
    assert cmds[1][0] == "ssh" and "--master-addr a" in cmds[1][-1] and "SUROGATE_NODE_RANK=1" in cmds[1][-1]
    monkeypatch.setenv("SLURM_NODEID", "3")
    assert d.node_rank_from_env() == 3
    name = d.detect_nccl_interface("127.0.0.1")
    assert name is None or isinstance(name, str)


def test_reporters_and_plot(tmp_path):
    from surogate_b200.train.reporter import make_reporters
    from surogate_b200.train.training_plot import plot_run, sparkline

    reps = make_reporters(["surogate", "wandb_not_installed_xyz"], "run", metrics_path=str(tmp_path / "m.jsonl"))
    assert len(reps) == 1
    log = tmp_path / "log.json"
    with open(log, "w") as f:
        for i in range(20):
            reps[0].log(i + 1, {"log": "step", "loss": 3.0 - 0.1 * i})
            f.write(json.dumps({"log": "step", "step": i + 1, "loss": 3.0 - 0.1 * i, "lr": 1e-3, "tps": 1000.0}) + "\n")
    reps[0].finish()
    assert len(open(tmp_path / "m.jsonl").read().splitlines()) == 20
    assert len(sparkline(list(range(100)), 40)) == 40
    assert "3.000 -> 1.100" in plot_run(str(log))


def test_regression_harness_detects_a_changed_loss():
    from surogate_b200.regression.runner import compare, default_matrix, run_case

    case = next(c for c in default_matrix(False) if c.name == "dense-bf16-adamw")
    case.steps = 3
    a, b = run_case(case), run_case(case)
    assert compare(a, b, time_factor=100.0) == []
    b["losses"][1] *= 1.2
    assert any("loss[1]" in p for p in compare(a, b, time_factor=100.0))


def test_locked_regression_baselines_still_hold():
    """The committed artifacts (regression_baselines/locked) against a fresh run of the same cases: losses, layout, parameter count."""
    from surogate_b200.regression.runner import compare, default_matrix, run_case

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "regression_baselines", "locked")
    assert len([f for f in os.listdir(root) if f.endswith(".json")]) >= 7
    for name in ("dense-bf16-adamw", "moe-bf16"):
        case = next(c for c in default_matrix(False) if c.name == name)
        with open(os.path.join(root, name + ".json")) as f:
            base = json.load(f)
        assert compare(run_case(case), base, time_factor=1e9, mem_factor=1e9) == [], name


def test_sft_workflow_with_adapter_resume(tmp_path):
    from surogate_b200.config.sft_config import SFTConfig
    from surogate_b200.train.sft import run_training

    model = dict(architecture="Qwen3ForCausalLM", vocab_size=256, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64,
                 tie_word_embeddings=True)
    base = dict(model=json.dumps(model), synthetic_data=True, sequence_len=32, per_device_train_batch_size=2, gradient_accumulation_steps=1, max_steps=3,
                lora=True, lora_rank=4, lora_alpha=8, optimizer="adamw", learning_rate=1e-2, save_steps=0, eval_steps=0, recipe="bf16", zero_level=0,
                from_scratch=False, report_to=["surogate"], surogate_metrics_path=str(tmp_path / "metrics.jsonl"))
    r1 = run_training(SFTConfig.from_dict(dict(base, output_dir=str(tmp_path / "a"))))
    assert r1["steps"] == 3 and os.path.exists(tmp_path / "a" / "adapter" / "adapter_model.safetensors")
    r2 = run_training(SFTConfig.from_dict(dict(base, output_dir=str(tmp_path / "b"), adapter_path=str(tmp_path / "a" / "adapter"), adapter_init_mode="resume")))
    assert r2["steps"] == 3 and np.isfinite(r2["final"]["loss"])
    assert os.path.getsize(tmp_path / "metrics.jsonl") > 0
    # ``trainable`` = resume with the parent checked against this run's LoRA settings
    r3 = run_training(SFTConfig.from_dict(dict(base, output_dir=str(tmp_path / "c"), adapter_path=str(tmp_path / "a" / "adapter"), adapter_init_mode="trainable")))
    assert r3["steps"] == 3 and abs(r3["losses"][0] - r2["losses"][0]) < 1e-6
    with pytest.raises(ValueError, match="rank"):
        run_training(SFTConfig.from_dict(dict(base, lora_rank=8, output_dir=str(tmp_path / "d"), adapter_path=str(tmp_path / "a" / "adapter"), adapter_init_mode="trainable")))
    os.remove(tmp_path / "a" / "adapter" / "adapter_config.json")
    with pytest.raises(FileNotFoundError, match="adapter_config.json"):
        run_training(SFTConfig.from_dict(dict(base, output_dir=str(tmp_path / "e"), adapter_path=str(tmp_path / "a" / "adapter"), adapter_init_mode="merge")))


def test_ray_launcher_places_one_task_per_node_on_a_stand_in_ray(monkeypatch):
    """``launch_with_ray`` against a minimal stand-in of the Ray API (Ray is not installed here): one bundle per node, strict spread,
    node 0's address as rendezvous address, one launcher command per bundle, placement group removed at the end."""
    import subprocess
    import sys
    import types

    log = {"bundles": None, "strategy": None, "placed": [], "removed": False}

    class _Remote:
        def __init__(self, fn, bundle=None):
            self.fn, self.bundle = fn, bundle

        def options(self, scheduling_strategy=None, **_):
            return _Remote(self.fn, scheduling_strategy.placement_group_bundle_index)

        def remote(self, *a):
            log["placed"].append((self.fn.__name__, self.bundle))
            return self.fn(*a)

    ray = types.ModuleType("ray")
    ray.init = lambda **kw: None
    ray.get = lambda x: x
    ray.remote = lambda **kw: (lambda fn: _Remote(fn))
    util = types.ModuleType("ray.util")
    util.get_node_ip_address = lambda: "10.1.2.3"
    pgm = types.ModuleType("ray.util.placement_group")

    class _PG:
        def ready(self):
            return True

    def placement_group(bundles, strategy):
        log["bundles"], log["strategy"] = bundles, strategy
        return _PG()

    pgm.placement_group = placement_group
    pgm.remove_placement_group = lambda pg: log.__setitem__("removed", True)
    ss = types.ModuleType("ray.util.scheduling_strategies")

    class PlacementGroupSchedulingStrategy:
        def __init__(self, placement_group, placement_group_bundle_index):
            self.placement_group, self.placement_group_bundle_index = placement_group, placement_group_bundle_index

    ss.PlacementGroupSchedulingStrategy = PlacementGroupSchedulingStrategy
    ray.util = util
    for name, mod in (("ray", ray), ("ray.util", util), ("ray.util.placement_group", pgm), ("ray.util.scheduling_strategies", ss)):
        monkeypatch.setitem(sys.modules, name, mod)
    calls = []
    monkeypatch.setattr(subprocess, "call", lambda cmd, env=None: calls.append((cmd, env)) or 0)
    from surogate_b200.train import distributed as d

    rcs = d.launch_with_ray("cfg.yaml", "sft", num_nodes=3, gpus_per_node=8, master_port=29555)
    assert rcs == [0, 0, 0] and log["removed"] and log["strategy"] == "STRICT_SPREAD" and log["bundles"] == [{"GPU": 8, "CPU": 1}] * 3
    assert log["placed"] == [("node_ip", 0), ("node_task", 0), ("node_task", 1), ("node_task", 2)]
    for node, (cmd, env) in enumerate(calls):
        assert f"--node-rank={node}" in cmd and "--nnodes=3" in cmd and cmd[cmd.index("--master-addr") + 1] == "10.1.2.3" and env["SUROGATE_NODE_RANK"] == str(node)

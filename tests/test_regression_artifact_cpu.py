"""``SUROGATE_REGRESSION_ARTIFACT``: a training run writes its convergence curve, timings and plan summary; two runs compare."""
import copy
import json

from surogate_b200.config.sft_config import SFTConfig
from surogate_b200.regression.artifact import RunArtifact, compare_runs, percentile_summary
from surogate_b200.train.sft import run_training

MODEL = dict(architecture="Qwen3ForCausalLM", vocab_size=96, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64, tie_word_embeddings=True)


def test_percentiles_and_env():
    s = percentile_summary([float(i) for i in range(1, 101)])
    assert s["count"] == 100 and s["min"] == 1 and s["max"] == 100 and s["p50"] == 51 and s["p95"] == 96 and percentile_summary([]) == {}
    assert RunArtifact.from_env({}) is None and RunArtifact.from_env({"SUROGATE_REGRESSION_ARTIFACT": "/x/a.json"}).path == "/x/a.json"


def test_a_run_writes_the_artifact(tmp_path, monkeypatch):
    path = tmp_path / "art" / "run.json"
    monkeypatch.setenv("SUROGATE_REGRESSION_ARTIFACT", str(path))
    cfg = SFTConfig.from_dict(dict(model=json.dumps(MODEL), synthetic_data=True, sequence_len=16, per_device_train_batch_size=2, gradient_accumulation_steps=1, max_steps=3,
                                   lora=False, optimizer="adamw", learning_rate=1e-2, save_steps=0, eval_steps=0, recipe="bf16", zero_level=0, from_scratch=True,
                                   output_dir=str(tmp_path / "run")))
    r = run_training(cfg)
    art = json.load(open(path))
    assert art["schema_version"] == 1 and [c["step"] for c in art["convergence_curve"]] == [1.0, 2.0, 3.0]
    assert [c["loss"] for c in art["convergence_curve"]] == r["losses"] and all(c["lr"] > 0 and c["grad_norm"] > 0 for c in art["convergence_curve"])
    assert art["step_time_ms"]["count"] == 2 and art["cuda_peak_memory_bytes"] is None and art["descriptor_summary"]["num_parameters"] > 0
    assert art["buffer_plan_summary"].get("saved_bytes", 0) > 0
    for key in ("activation_snapshots", "gradient_snapshots", "nccl", "block_schema_summary"):
        assert key in art
    assert compare_runs(art, art) == []
    worse = copy.deepcopy(art)
    worse["convergence_curve"][1]["loss"] *= 1.5
    worse["step_time_ms"]["p50"] *= 3
    worse["buffer_plan_summary"]["saved_bytes"] += 4096
    problems = compare_runs(worse, art)
    assert len(problems) == 3 and "loss at step 2" in problems[0] and "step time" in problems[1] and "buffer_plan_summary" in problems[2]
    assert "step count" in compare_runs(dict(art, convergence_curve=art["convergence_curve"][:2]), art)[0]


def test_config_harness_runs_a_subprocess_and_compares(tmp_path, capsys):
    import yaml

    from surogate_b200.regression.runner import main

    cfg = dict(model=json.dumps(MODEL), synthetic_data=True, sequence_len=16, per_device_train_batch_size=2, gradient_accumulation_steps=1, max_steps=2, lora=False,
               optimizer="adamw", learning_rate=1e-2, save_steps=0, eval_steps=0, recipe="bf16", zero_level=0, from_scratch=True, output_dir=str(tmp_path / "run"))
    path = tmp_path / "tiny.yaml"
    path.write_text(yaml.safe_dump(cfg))
    base = str(tmp_path / "baselines")
    assert main(["--baselines", base, "--config", str(path)]) == 0 and "[baseline] tiny" in capsys.readouterr().out
    art = json.load(open(tmp_path / "baselines" / "tiny.json"))
    assert len(art["convergence_curve"]) == 2
    assert main(["--baselines", base, "--config", str(path)]) == 0 and "[ ok ] tiny" in capsys.readouterr().out  # same seeds, same curve
    art["convergence_curve"][0]["loss"] += 1.0
    json.dump(art, open(tmp_path / "baselines" / "tiny.json", "w"))
    assert main(["--baselines", base, "--config", str(path)]) == 1 and "loss at step 1" in capsys.readouterr().out
    bad = tmp_path / "bad.yaml"
    bad.write_text("model: /nonexistent/model/dir\n")
    assert main(["--baselines", base, "--config", str(bad)]) == 1 and "[FAIL] bad" in capsys.readouterr().out

"""The parts of bench.py's contract that need no GPU: flags and defaults, the reference arm's one-line answer, the model table."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_and_exits_zero():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and len(d["unavailable"]) > 20


def test_flags_defaults_and_model_table():
    sys.path.insert(0, ROOT)
    try:
        import bench
    finally:
        sys.path.pop(0)
    old = sys.argv
    sys.argv = ["bench.py"]
    try:
        a = bench.parse_args()
    finally:
        sys.argv = old
    assert a.gpus == 1 and a.impl == "native" and a.model == "qwen3-8b" and a.steps >= 1 and a.ep_refresh == 0 and not a.no_secondary
    m = bench.MODELS
    assert set(m) >= {"qwen3-8b", "qwen3-30b-a3b", "qwen3-0.6b", "qwen3-14b-lora"}
    q8 = m["qwen3-8b"]
    assert q8["recipe"] == "fp8_hybrid" and q8["zero"] == 3 and q8["seq_len"] == 4096 and q8["batch"] == 2 and q8["optimizer"] == "adamw_8bit"
    assert q8["model"]["n_layers"] == 36 and q8["model"]["d_model"] == 4096 and q8["model"]["vocab_size"] == 151936
    moe = m["qwen3-30b-a3b"]
    assert moe["recipe"] == "nvfp4" and moe["model"]["num_experts"] == 128 and moe["model"]["num_experts_per_tok"] == 8 and moe["seq_len"] == 4096 and moe["batch"] == 1

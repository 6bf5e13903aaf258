"""CLI plumbing and offline tools on CPU: export -> audit -> merge -> debug stats; tokenise pipeline; every command imports."""
import importlib
import json
import os

import numpy as np
import pytest
import torch

from surogate_b200.runtime.trainer import Trainer, TrainerConfig

MODEL = dict(architecture="Qwen3ForCausalLM", vocab_size=600, d_model=32, n_layers=2, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64,
             tie_word_embeddings=False)
LORA = dict(rank=4, alpha=8, dropout=0.0, dtype="fp32", targets=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"],
            rslora=False, train_router=False)


def test_every_cli_command_module_imports():
    from surogate_b200.cli.main import COMMAND_MAPPING, cli_main

    for mod in set(COMMAND_MAPPING.values()):
        assert hasattr(importlib.import_module(mod), "main"), mod
    assert cli_main(["--help"]) == 0 and cli_main(["nonsense"]) == 2


def _trained_lora(tmp_path):
    tr = Trainer(TrainerConfig(model=MODEL, batch_size=2, seq_len=16, recipe="bf16", optimizer="adamw", learning_rate=5e-2, zero_level=0, lora=LORA),
                 device=torch.device("cpu"))
    tr.init_weights(seed=0)
    rng = np.random.default_rng(0)
    tok = rng.integers(0, 600, (2, 17)).astype(np.int32)
    for _ in range(3):
        tr.step(tok[:, :-1], tok[:, 1:])
    base, adapter = os.path.join(tmp_path, "base"), os.path.join(tmp_path, "adapter")
    tr.export_model(base, MODEL)
    tr.export_adapter(adapter, base_model=base)
    return tr, tok, base, adapter


def test_merge_adapter_on_safetensors_matches_in_memory_merge(tmp_path):
    from safetensors.torch import load_file

    from surogate_b200.cli.main import cli_main
    from surogate_b200.debug.tools import audit_weights

    tr, tok, base, adapter = _trained_lora(str(tmp_path))
    merged = os.path.join(tmp_path, "merged")
    assert cli_main(["merge", "--base", base, "--adapter", adapter, "--output", merged]) == 0
    tr.lora.merge_into(tr.store)
    ref = os.path.join(tmp_path, "ref")
    tr.export_model(ref, MODEL)
    a, b = load_file(os.path.join(merged, "model.safetensors")), load_file(os.path.join(ref, "model.safetensors"))
    assert a.keys() == b.keys()
    changed = 0
    base_t = load_file(os.path.join(base, "model.safetensors"))
    for k in a:
        assert torch.allclose(a[k].float(), b[k].float(), atol=2e-2, rtol=2e-2), k
        changed += int(not torch.equal(a[k], base_t[k]))
    assert changed >= 2 * 7  # every adapted projection of both layers moved
    rep = audit_weights(merged)
    assert rep["missing"] == [] and rep["unused"] == []


def test_debug_stats_and_registry(tmp_path):
    from surogate_b200.debug import tools

    tr, tok, base, _ = _trained_lora(str(tmp_path))
    acts = tools.activation_stats(tr, tok[:, :-1], tok[:, 1:], os.path.join(tmp_path, "acts.jsonl"))
    assert any(r["layer"] == 1 for r in acts) and all(r["nonfinite"] == 0 for r in acts)
    grads = tools.gradient_stats(tr, tok[:, :-1], tok[:, 1:])
    assert grads == [] or all("param" in g for g in grads)  # base is frozen under LoRA
    reg = tools.registry_report(base)
    assert "Qwen3ForCausalLM" in reg[0]["architectures"] and any(r.get("graph") == "forward" for r in reg)


def test_tokenize_pipeline_packs_and_caches(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    from test_host_runtime import QWEN_PATTERN, _train_tokenizer

    from surogate_b200.config.sft_config import SFTConfig
    from surogate_b200.data.tokfile import read_token_file
    from surogate_b200.train.tokenize import TokenizeDatasets

    _, mdir = _train_tokenizer(QWEN_PATTERN, str(tmp_path), "model")
    with open(os.path.join(mdir, "tokenizer_config.json"), "w") as f:
        json.dump({"eos_token": "<|im_end|>", "pad_token": "<|endoftext|>"}, f)
    data = os.path.join(tmp_path, "chat.jsonl")
    with open(data, "w") as f:
        for i in range(12):
            f.write(json.dumps({"messages": [{"role": "user", "content": f"Hello world {i}"}, {"role": "assistant", "content": "It's a test " * (1 + i % 3)}]}) + "\n")
    cfg = SFTConfig.from_dict(dict(model=mdir, datasets=[{"path": data}], sequence_len=64, output_dir=str(tmp_path / "out"), validation_split_ratio=0.25))
    job = TokenizeDatasets(cfg, {"vocab_size": 600}, os.path.join(tmp_path, "tok"))
    files = job.run()
    assert job.stats["train_documents"] == 9 and job.stats["eval_documents"] == 3
    assert job.stats["train_rows"] < job.stats["train_documents"]  # packing put several conversations into one row
    tok, pos, mask, h = read_token_file(files["train"][0])
    assert h["non_overlapping"] == 1 and h["has_masks"] == 1 and len(tok) == job.stats["train_rows"] * 64
    assert (pos[:64] == 0).sum() >= 2  # position ids restart per document
    assert 0 < mask.sum() < len(mask)  # only assistant tokens are trained
    again = TokenizeDatasets(cfg, {"vocab_size": 600}, os.path.join(tmp_path, "tok"))
    assert again.run() == files and not hasattr(again, "stats")  # served from the cache


def test_upcycle_quantize_and_generate(tmp_path):
    """Dense -> MoE upcycling keeps the function (every expert = the dense MLP, weights renormalised over top-k sum to 1);
    block-FP8 quantisation round-trips within FP8 error; the chat helper decodes greedily."""
    from safetensors.torch import load_file

    from surogate_b200.cli.chat import generate
    from surogate_b200.dsl.compiler import load_hf_config
    from surogate_b200.quant.codecs import BlockFP8
    from surogate_b200.utils.quantize_fp8 import quantize_checkpoint
    from surogate_b200.utils.upcycle_moe import upcycle

    dense = dict(MODEL)
    tr = Trainer(TrainerConfig(model=dense, batch_size=1, seq_len=16, zero_level=0), device=torch.device("cpu"))
    tr.init_weights(seed=0)
    src = os.path.join(tmp_path, "dense")
    tr.export_model(src, dense)
    moe_dir = os.path.join(tmp_path, "moe")
    info = upcycle(src, moe_dir, num_experts=4, top_k=2)
    assert info["experts"] == 4
    moe = Trainer(TrainerConfig(model=load_hf_config(moe_dir), batch_size=1, seq_len=16, zero_level=0), device=torch.device("cpu"))
    moe.import_weights(moe_dir)
    tok = np.random.default_rng(0).integers(0, 600, (1, 16)).astype(np.int32)
    a, b = tr.logits(tok), moe.logits(tok)
    assert torch.allclose(a, b, atol=2e-2, rtol=2e-2)  # bf16 export in between
    out = generate(tr, None, tok[0, :4].tolist(), max_new_tokens=5, eos_id=None)
    assert len(out) == 5 and all(0 <= t < 600 for t in out)
    # health check: fresh experts are clones and the near-zero router is close to random; noisy experts have diverged
    from surogate_b200.utils.expert_divergence import expert_divergence, verdict

    rep = expert_divergence(moe_dir, tokens=64)
    assert rep["num_experts"] == 4 and rep["expert_similarity"] > 0.9999 and rep["experts"].startswith("clones") and set(rep["projections"]) == {"gate_proj", "up_proj", "down_proj"}
    assert rep["router"]["random_level"] == 0.25 and rep["router"]["mean_top1_probability"] < 0.35
    noisy = os.path.join(tmp_path, "moe_noisy")
    upcycle(src, noisy, num_experts=4, top_k=2, noise=0.5)
    assert expert_divergence(noisy, layer=0, tokens=0)["expert_similarity"] < 0.99
    assert verdict(0.9995).startswith("barely") and verdict(0.5) == "specialised"
    with pytest.raises(ValueError, match="not a mixture-of-experts"):
        expert_divergence(src)
    q_dir = os.path.join(tmp_path, "fp8")
    rep = quantize_checkpoint(src, q_dir)
    assert rep["quantized"] == 2 * 7  # q, k, v, o, gate, up, down per layer; embeddings, norms and the head keep their dtype
    t = load_file(os.path.join(q_dir, "model.safetensors"))
    name = "model.layers.0.mlp.down_proj.weight"
    back = BlockFP8.dequantize_2d(t[name], t[name + "_scale_inv"], dtype=torch.float32)
    ref = load_file(os.path.join(src, "model.safetensors"))[name].float()
    assert ((back - ref).norm() / ref.norm()).item() < 0.05
    assert json.load(open(os.path.join(q_dir, "config.json")))["quantization_config"]["quant_method"] == "fp8"


def test_monitor_tails_the_metrics_feed(tmp_path, capsys):
    """The dashboard reads the feed incrementally (partial last lines wait, a truncated file restarts) and renders a frame."""
    from surogate_b200.cli import monitor

    feed = tmp_path / "metrics.jsonl"
    with open(feed, "w") as f:
        f.write(json.dumps({"log": "options", "config": {"run_name": "demo", "max_steps": 40}}) + "\n")
        for i in range(20):
            f.write(json.dumps({"log": "step", "step": i + 1, "loss": 3.0 - 0.1 * i, "lr": 1e-3, "norm": 1.5, "tps": 1000.0 + i}) + "\n")
        f.write(json.dumps({"log": "eval", "step": 20, "loss": 1.25}) + "\n")
        f.write(json.dumps({"log": "gpu", "index": 0, "gpu_util": 90, "mem_used": 2**34, "mem_total": 2**35}) + "\n")
        f.write('{"log": "step", "step": 21, "lo')  # writer is mid-line
    st = monitor.FeedState(str(feed))
    assert st.poll() == 23 and st.steps[-1] == 20 and st.max_steps == 40 and st.run_name == "demo"
    with open(feed, "a") as f:
        f.write('ss": 0.9, "lr": 0.001, "norm": 1.0, "tps": 1100.0}\n')
    assert st.poll() == 1 and st.steps[-1] == 21 and abs(st.series["loss"][-1] - 0.9) < 1e-9
    frame = monitor.render(st, 100)
    assert "TRAINING LOSS" in frame and "step 21/40" in frame and "gpu0" in frame and "EVAL" in frame and "demo" in frame
    rows = monitor.chart([3.0, 2.0, 1.0], 10, 4)
    assert len(rows) == 4 and "█" in rows[-1]
    with open(feed, "w") as f:
        f.write(json.dumps({"log": "step", "step": 1, "loss": 5.0, "lr": 1e-3, "norm": 1.0, "tps": 10.0}) + "\n")
    assert st.poll() == 1 and st.steps == [1]
    assert monitor.main(["--feed", str(feed), "--once"]) == 0
    assert "TRAINING LOSS" in capsys.readouterr().out


def test_every_example_configuration_loads_and_validates():
    """The shipped example YAML files parse into their config classes and pass validation."""
    import glob

    import yaml

    from surogate_b200.config.sft_config import SFTConfig
    from surogate_b200.dpo.config import DPOConfig
    from surogate_b200.grpo.config import GRPOConfig, InferenceConfig, OrchestratorConfig

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
    files = sorted(glob.glob(os.path.join(root, "**", "*.yaml"), recursive=True))
    assert len(files) >= 15
    for f in files:
        d = yaml.safe_load(open(f))
        rel = os.path.relpath(f, root)
        if rel.startswith("dpo"):
            cfg = DPOConfig.from_dict(d)
        elif rel == os.path.join("grpo", "train.yaml"):
            cfg = GRPOConfig.from_dict(d)
        elif rel in (os.path.join("grpo", "infer.yaml"), os.path.join("ruler", "judge.yaml")):
            cfg = InferenceConfig(**d)
        elif rel == os.path.join("grpo", "orch.yaml"):
            cfg = OrchestratorConfig(**d)
        elif rel == os.path.join("ruler", "orch.yaml"):
            from surogate_b200.grpo.ruler import RulerConfig

            cfg = OrchestratorConfig(**d)
            assert RulerConfig.from_dict(cfg.ruler).mode == "replace" and cfg.rows_per_step == 0
        elif rel == os.path.join("grpo", "orch-async.yaml"):
            from surogate_b200.grpo.orchestration import async_config_from, make_filters
            from surogate_b200.grpo.orchestration.buffer import BufferConfig
            from surogate_b200.grpo.orchestration.depth import RolloutDepthController

            cfg = OrchestratorConfig(**{k: v for k, v in d.items() if k in OrchestratorConfig.__dataclass_fields__})
            a = async_config_from(cfg, d, vocab_size=1000)
            assert a.batch_size == 128 and a.max_inflight == 48 and len(make_filters(a.filters, 1000)) == 2 and d["scheduler"] == "async"
            assert BufferConfig(**a.buffer).min_normal == 256 and RolloutDepthController(**a.depth).max_cap == 24
        else:
            cfg = SFTConfig.from_dict(d)
        assert cfg.model, rel
        if hasattr(cfg, "to_trainer_config") and not rel.startswith("grpo"):
            hf = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=64, num_hidden_layers=8, num_attention_heads=4, num_key_value_heads=2,
                      head_dim=16, intermediate_size=96, vocab_size=320)
            assert cfg.to_trainer_config(hf).seq_len == cfg.sequence_len, rel


def test_eval_command_reports_loss_and_perplexity(tmp_path, capsys):
    import yaml

    from surogate_b200.cli.main import cli_main

    model = dict(architecture="Qwen3ForCausalLM", vocab_size=256, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64,
                 tie_word_embeddings=True)
    cfg = dict(model=json.dumps(model), synthetic_data=True, sequence_len=32, per_device_train_batch_size=2, output_dir=str(tmp_path / "out"), lora=False,
               recipe="bf16", zero_level=0)
    path = tmp_path / "cfg.yaml"
    path.write_text(yaml.safe_dump(cfg))
    os.environ["SUROGATE_NO_BANNER"] = "1"
    assert cli_main(["eval", str(path), "--batches", "2"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["batches"] == 2 and 4.0 < out["eval_loss"] < 7.0 and abs(out["perplexity"] - np.exp(out["eval_loss"])) < 1e-6 * out["perplexity"]


def test_object_store_datasets_are_fetched_through_fsspec(tmp_path, monkeypatch):
    """Any fsspec URL works as a dataset path (memory:// stands in for s3:// / gs://): files are cached locally and parsed."""
    import fsspec

    from surogate_b200.config.sft_config import DatasetConfig
    from surogate_b200.data.datasets import fetch_remote, load_rows

    fs = fsspec.filesystem("memory")
    with fs.open("/bucket/set/train-0.jsonl", "w") as f:
        f.write("\n".join(json.dumps({"text": f"row {i}"}) for i in range(5)))
    with fs.open("/bucket/set/eval-0.jsonl", "w") as f:
        f.write(json.dumps({"text": "held out"}))
    monkeypatch.setenv("SUROGATE_CACHE", str(tmp_path))
    rows = load_rows(DatasetConfig(path="memory://bucket/set", type="text", split="train"))
    assert [r["text"] for r in rows] == [f"row {i}" for i in range(5)]
    again = fetch_remote("memory://bucket/set/eval-0.jsonl")
    assert len(again) == 1 and os.path.getsize(again[0]) > 0 and fetch_remote("memory://bucket/set/eval-0.jsonl") == again
    try:
        load_rows(DatasetConfig(path="nosuchproto://x/y"))
        raise AssertionError("expected an error for an unknown protocol")
    except RuntimeError as e:
        assert "fsspec backend" in str(e)


def test_determinism_report_and_sanitized_host_runtime():
    """Two runs from the same seed agree bit for bit on the PyTorch backend; the host runtime's built-in workload is clean under
    AddressSanitizer + UBSan (skipped where gcc has no sanitizer runtime)."""
    import subprocess
    import sys

    from surogate_b200.debug import sanitize, tools

    def make():
        tr = Trainer(TrainerConfig(model=dict(MODEL), batch_size=1, seq_len=16, zero_level=0), device=torch.device("cpu"))
        tr.init_weights(seed=0)
        return tr

    tok = np.random.default_rng(0).integers(0, 600, (1, 17)).astype(np.int32)
    rep = tools.determinism_report(make, tok[:, :-1], tok[:, 1:], steps=2)
    assert rep["bitwise_equal"] and rep["n_params"] > 5 and rep["steps"][0]["loss_a"] == rep["steps"][0]["loss_b"]
    rt = sanitize.sanitizer_runtime()
    if rt is None:
        return
    from surogate_b200.ops import _build

    so = _build.build_host_sanitized()
    env = dict(os.environ, LD_PRELOAD=rt, SUROGATE_HOST_SO=so, ASAN_OPTIONS="detect_leaks=0:halt_on_error=1", UBSAN_OPTIONS="halt_on_error=1", OMP_NUM_THREADS="2")
    p = subprocess.run([sys.executable, "-c", "from surogate_b200.debug.sanitize import builtin_workload; builtin_workload()"], env=env, capture_output=True,
                       text=True, timeout=600, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert p.returncode == 0 and "host workload ok" in p.stdout, p.stderr[-3000:]
    assert "ERROR: AddressSanitizer" not in p.stderr and "runtime error" not in p.stderr


def test_dashboard_browses_models_datasets_and_runs(tmp_path, capsys):
    """The dashboard's Models / Datasets / Runs views: local model directories with the 'trainable' badge from the architecture
    registry, a hub search through an injected function, dataset files with their detected type, and past runs of an output root."""
    import json

    from surogate_b200.cli import monitor

    (tmp_path / "models" / "a").mkdir(parents=True)
    (tmp_path / "models" / "b").mkdir()
    (tmp_path / "models" / "a" / "config.json").write_text(json.dumps({"architectures": ["Qwen3ForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2}))
    (tmp_path / "models" / "b" / "config.json").write_text(json.dumps({"architectures": ["SomethingElseForCausalLM"], "num_experts": 4}))
    rows = monitor.browse_models(str(tmp_path / "models"))
    assert [(os.path.basename(r["id"]), r["trainable"], r["moe"]) for r in rows] == [("a", True, False), ("b", False, True)]
    hub = monitor.browse_models("qwen", search=lambda q, n: [{"id": "org/m1", "architectures": ["Qwen3MoeForCausalLM"], "downloads": 5},
                                                              {"id": "org/m2", "architectures": ["BertModel"]}])
    assert [(r["id"], r["trainable"]) for r in hub] == [("org/m1", True), ("org/m2", False)]

    (tmp_path / "data").mkdir()
    (tmp_path / "data" / "chat.jsonl").write_text(json.dumps({"messages": [{"role": "user", "content": "hi"}]}) + "\n")
    (tmp_path / "data" / "pairs.jsonl").write_text(json.dumps({"prompt": "p", "chosen": "a", "rejected": "b"}) + "\n")
    ds = {os.path.basename(r["id"]): r["type"] for r in monitor.browse_datasets(str(tmp_path / "data"))}
    assert ds == {"chat.jsonl": "messages", "pairs.jsonl": "preference"}
    assert monitor.browse_datasets("x", search=lambda q, n: [{"id": "org/d", "downloads": 3}]) == [{"id": "org/d", "downloads": 3}]

    run = tmp_path / "out" / "run1"
    (run / "step_00000010").mkdir(parents=True)
    (run / "log.jsonl").write_text("".join(json.dumps({"log": "step", "step": i, "loss": 3.0 - 0.1 * i}) + "\n" for i in range(1, 11)))
    runs = monitor.past_runs(str(tmp_path / "out"))
    assert runs == [{"run": "run1", "step": 10, "loss": 2.0, "checkpoints": 1, "exported": False}]
    assert monitor.main(["runs", str(tmp_path / "out")]) == 0
    assert "run1" in capsys.readouterr().out


def test_config_values_written_as_text_reach_their_declared_type(tmp_path, monkeypatch):
    """`learning_rate: 3e-4` (a string for YAML 1.1) and `${ENV}` expansions become numbers / booleans of the field's type; text
    that does not parse names the key."""
    import pytest

    from surogate_b200.config.loader import load_config
    from surogate_b200.config.sft_config import SFTConfig

    monkeypatch.setenv("MY_STEPS", "12")
    p = tmp_path / "c.yaml"
    p.write_text("model: m\nlearning_rate: 3e-4\nmax_steps: ${MY_STEPS}\nrecompute: 'false'\nweight_decay: 1\nwarmup_ratio: '0.1'\n")
    c = load_config(SFTConfig, str(p))
    assert c.learning_rate == 3e-4 and isinstance(c.learning_rate, float)
    assert c.max_steps == 12 and c.recompute is False and isinstance(c.weight_decay, float) and c.warmup_ratio == 0.1
    p.write_text("model: m\nlearning_rate: fast\n")
    with pytest.raises(ValueError, match="learning_rate"):
        load_config(SFTConfig, str(p))


def test_metrics_feed_uses_the_dashboard_schema_and_the_monitor_reads_it(tmp_path, monkeypatch):
    """The feed's records carry the dashboard's field names (``train/loss``, ``type: gpu`` ...), the monitor reads them, and the
    feed path falls back to the environment variable a launcher sets."""
    from surogate_b200.cli import monitor
    from surogate_b200.train.logging import TrainingRunLogger, feed_record, resolve_metrics_path

    feed = tmp_path / "feed.jsonl"
    monkeypatch.setenv("SUROGATE_METRICS_PATH", str(feed))
    assert resolve_metrics_path("/tmp/surogate_metrics.jsonl") == str(feed)
    assert resolve_metrics_path(str(tmp_path / "explicit.jsonl")) == str(tmp_path / "explicit.jsonl")

    import io

    lg = TrainingRunLogger(None, resolve_metrics_path(None), stream=io.StringIO())
    lg.log_record("options", config={"run_name": "r1", "model": "Qwen/Qwen3-0.6B", "recipe": "fp8-hybrid", "max_steps": 10, "nested": {"a": 1}})
    for i in range(3):
        lg.log_step(i + 1, 10, 0.1 * i, 3.0 - i, 1.5, 1e-3, 8192, 100.0, phase="converging")
    lg.log_eval(3, 2.5)
    lg.log_record("gpu", step=3, name="B200", temperature_c=55, power_w=700.0, gpu_util=97, mem_util=40, mem_used=2**30, mem_total=2**31)
    lg.log_record("moe", step=3, imbalance=1.5, aux_loss=0.01)
    lg.message("not part of the feed")
    lg.close()
    recs = [json.loads(l) for l in open(feed)]
    assert len(recs) == 7
    cfg, s1, ev, gpu = recs[0], recs[1], recs[4], recs[5]
    assert cfg["type"] == "config" and cfg["model"] == "Qwen/Qwen3-0.6B" and cfg["recipe"] == "fp8-hybrid" and "nested" not in cfg
    assert "type" not in s1 and s1["step"] == 1 and s1["train/loss"] == 3.0 and s1["train/norm"] == 1.5 and s1["train/lr"] == 1e-3
    assert abs(s1["train/tokens_per_second"] - 81920.0) < 1e-6 and s1["train/phase"] == "converging" and "ts" in s1
    assert ev["eval/loss"] == 2.5 and "train/loss" not in ev
    assert gpu["type"] == "gpu" and gpu["gpu_id"] == 0 and gpu["temperature"] == 55 and gpu["power"] == 700.0 and gpu["gpu_utilization"] == 97
    assert feed_record({"log": "message", "text": "x"}) is None

    st = monitor.FeedState(str(feed))
    assert st.poll() == 7
    assert st.steps == [1, 2, 3] and st.series["loss"] == [3.0, 2.0, 1.0] and st.max_steps == 10 and st.run_name == "r1"
    assert st.evals == [(3, 2.5)] and st.gpu["gpu_util"] == 97 and st.moe["imbalance"] == 1.5
    frame = monitor.render(st, width=100)
    assert "step 3/10" in frame and "MoE" in frame and "gpu0" in frame


def test_tokenisation_lock_serialises_two_writers(tmp_path):
    """Two processes that want to write shards into the same directory: the second enters only after the first has left."""
    import subprocess
    import sys
    import time

    from surogate_b200.train.tokenize import directory_lock, progress

    d = str(tmp_path)
    child = (f"import sys, time; sys.path.insert(0, {os.getcwd()!r}); from surogate_b200.train.tokenize import directory_lock\n"
             f"with directory_lock({d!r}):\n    open({os.path.join(d, 'child_in')!r}, 'w').write(str(time.time()))\n")
    with directory_lock(d):
        p = subprocess.Popen([sys.executable, "-c", child])
        time.sleep(1.5)
        assert not os.path.exists(os.path.join(d, "child_in"))      # blocked while this process holds the lock
        released = time.time()
    assert p.wait(timeout=60) == 0 and float(open(os.path.join(d, "child_in")).read()) >= released - 0.05
    assert list(progress(iter(range(3)), "x")) == [0, 1, 2]

"""Command lines written for the reference work here: the argument forms of ``grpo`` / ``grpo-train``, ``merge``, ``tokenize``,
``vf-eval``, ``--hub_token``, the ``jackalope`` command."""
import json
import os
import threading
from http.server import BaseHTTPRequestHandler, HTTPServer

import pytest
import torch
import yaml

from surogate_b200.cli.main import COMMAND_MAPPING, cli_main


def _tiny_model():
    return dict(architecture="Qwen3ForCausalLM", vocab_size=96, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64, tie_word_embeddings=True)


def test_grpo_and_grpo_train_accept_either_form(tmp_path, capsys, monkeypatch):
    from surogate_b200.cli import grpo as cli

    assert cli.is_supervised(["--train", "t.yaml"]) and cli.is_supervised(["--orch", "o", "--train=t.yaml"]) and not cli.is_supervised(["t.yaml", "--max-steps", "3"])
    for name, body in (("t.yaml", {"model": "m", "gpus": 2}), ("i.yaml", {"model": "m", "tensor_parallel_size": 1}), ("o.yaml", {"model": "m"}), ("j.yaml", {"model": "judge"})):
        (tmp_path / name).write_text(yaml.safe_dump(body))
    common = ["--train", str(tmp_path / "t.yaml"), "--infer", str(tmp_path / "i.yaml"), "--orch", str(tmp_path / "o.yaml"), "--dry-run"]
    monkeypatch.setenv("SUROGATE_NO_BANNER", "1")
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    outs = {}
    for cmd in ("grpo", "grpo-train"):  # the split-GPU run under both names
        assert cli_main([cmd, *common, "--trainer-gpus", "0,1", "--vllm-gpus", "2", "--judge-infer", str(tmp_path / "j.yaml"), "--judge-gpus", "3"]) == 0
        outs[cmd] = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert outs["grpo"] == outs["grpo-train"]
    comps = {c["name"]: c for c in outs["grpo"]}
    assert set(comps) == {"rollout engine", "judge engine", "orchestrator", "trainer"}
    assert comps["rollout engine"]["env"]["CUDA_VISIBLE_DEVICES"] == "2" and comps["judge engine"]["env"]["CUDA_VISIBLE_DEVICES"] == "3"
    assert comps["trainer"]["env"]["CUDA_VISIBLE_DEVICES"] == "0,1" and "CUDA_VISIBLE_DEVICES" not in os.environ  # the supervisor itself is not masked
    assert cli_main(["grpo-colocate", *common, "--gpus", "0,1"]) == 0
    assert {json.loads(l)["name"] for l in capsys.readouterr().out.strip().splitlines()} == {"rollout engine", "orchestrator", "trainer"}
    # the trainer alone, under both names: one positional config
    seen = []
    import surogate_b200.grpo.trainer as trainer_mod

    monkeypatch.setattr(trainer_mod, "run_grpo", lambda cfg: seen.append(cfg) or {"steps": 0, "history": []})
    import surogate_b200.config.loader as loader

    monkeypatch.setattr(loader, "load_config", lambda cls, path, **kw: (cls.__name__, path, kw))
    for cmd in ("grpo", "grpo-train"):
        assert cli_main([cmd, str(tmp_path / "t.yaml"), "--max-steps", "3", "--trainer-gpus", "5"]) == 0
        assert os.environ.pop("CUDA_VISIBLE_DEVICES") == "5"
    capsys.readouterr()
    assert seen == [("GRPOConfig", str(tmp_path / "t.yaml"), {"max_steps": 3})] * 2


def test_merge_accepts_the_checkpoint_dir_spelling(tmp_path, capsys):
    from safetensors.torch import save_file

    from surogate_b200.cli import merge as cli

    base, run = tmp_path / "base", tmp_path / "run"
    os.makedirs(base)
    os.makedirs(run / "adapter")
    W = torch.randn(8, 8)
    save_file({"model.layers.0.self_attn.q_proj.weight": W}, str(base / "model.safetensors"), metadata={"format": "pt"})
    (base / "config.json").write_text("{}")
    A, B = torch.randn(2, 8), torch.randn(8, 2)
    save_file({"base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight": A, "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight": B},
              str(run / "adapter" / "adapter_model.safetensors"))
    (run / "adapter" / "adapter_config.json").write_text(json.dumps({"r": 2, "lora_alpha": 4, "target_modules": ["q_proj"]}))
    # --checkpoint-dir may name the run directory that holds adapter/
    assert cli.main(["--base-model", str(base), "--checkpoint-dir", str(run), "--output", str(tmp_path / "m1")]) == 0
    assert cli.main(["--base", str(base), "--adapter", str(run / "adapter"), "--output", str(tmp_path / "m2")]) == 0
    capsys.readouterr()
    from safetensors import safe_open

    for m in ("m1", "m2"):
        with safe_open(str(tmp_path / m / "model.safetensors"), framework="pt") as f:
            got = f.get_tensor("model.layers.0.self_attn.q_proj.weight")
        assert torch.allclose(got, W + 2.0 * (B @ A), atol=1e-5)


def test_tokenize_debug_prints_tokens_with_their_labels(tmp_path, capsys):
    from surogate_b200.cli import tokenize as cli

    cfg = dict(model=json.dumps(_tiny_model()), synthetic_data=False, sequence_len=16, per_device_train_batch_size=2, output_dir=str(tmp_path / "run"))
    from surogate_b200.data.tokfile import TokenFileWriter
    import numpy as np

    shard = str(tmp_path / "train-000.bin")
    w = TokenFileWriter(shard, 96, has_masks=True, non_overlapping=True)
    ids = np.arange(16, dtype=np.int32)
    mask = np.array([0] * 6 + [1] * 10, np.uint8)
    try:
        w.add(ids, position_ids=np.arange(16, dtype=np.int32), mask=mask)
    except TypeError:
        w.add(ids, np.arange(16, dtype=np.int32), mask)
    w.close()
    text = cli.debug_rows(shard, None, 16)
    lines = text.splitlines()
    assert lines[0] == "--- row 0: 10 of 16 tokens trained" and lines[1].split()[-1] == "-" and lines[7].split()[-1] == "train" and len(lines) == 17
    assert cfg  # the command-line flag itself is declared
    with pytest.raises(SystemExit):
        cli.main(["--help"])
    assert "--debug" in capsys.readouterr().out


def test_vf_eval_options(tmp_path, capsys, monkeypatch):
    from surogate_b200.cli import vf as cli

    seen = {"bodies": [], "headers": [], "fail_first": True}
    lock = threading.Lock()

    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            with lock:
                fail, seen["fail_first"] = seen["fail_first"], False
                seen["bodies"].append(body)
                seen["headers"].append({k.lower(): v for k, v in self.headers.items()})
            if fail:
                self.send_response(500)
                self.end_headers()
                return
            data = json.dumps({"choices": [{"message": {"content": "42"}}]}).encode()
            self.send_response(200)
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

    srv = HTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        pkg = tmp_path / "envs" / "my_env"
        os.makedirs(pkg)
        (pkg / "__init__.py").write_text(
            "from surogate_b200.grpo.environments.base import SingleTurnEnv, Rubric\n"
            "def exact(completion, answer, **_):\n"
            "    return float(completion.strip() == answer)\n"
            "def load_environment(n=3, **_):\n"
            "    data = [{'prompt': [{'role': 'user', 'content': f'q{i}'}], 'answer': '42'} for i in range(n)]\n"
            "    env = SingleTurnEnv(data, Rubric([exact], [1.0]))\n"
            "    env.env_id = 'my-env'\n"
            "    return env\n")
        monkeypatch.setenv("MY_KEY", "sekret")
        save = tmp_path / "res.json"
        rc = cli.main(["my-env", "--env-path", str(tmp_path / "envs"), "-a", '{"n": 4}', "-m", "served", "--api-base-url", f"http://127.0.0.1:{srv.server_port}/v1",
                       "--api-key-var", "MY_KEY", "--header", "X-Run: r1", "-n", "4", "-r", "2", "-c", "4", "-t", "64", "-T", "0.5", "-S", '{"top_p": 0.9}',
                       "--max-retries", "2", "--save-results", str(save), "-v"])
        assert rc == 0
    finally:
        srv.shutdown()
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["n"] == 8 and out["mean_reward"] == 1.0 and "samples" not in out and len(json.load(open(save))["samples"]) == 8
    ok = [b for b in seen["bodies"]]
    assert len(ok) == 9  # 8 rollouts + the one retried failure
    assert all(b["model"] == "served" and b["top_p"] == 0.9 and b["max_tokens"] == 64 and b["temperature"] == 0.5 for b in ok)
    assert all(h["authorization"] == "Bearer sekret" and h["x-run"] == "r1" for h in seen["headers"])
    with pytest.raises(SystemExit):
        cli.main(["my-env", "--header", "broken"])


def test_hub_token_and_dashboard_alias(monkeypatch):
    from surogate_b200.cli.sft import build_parser, take_hub_token

    assert COMMAND_MAPPING["jackalope"] == COMMAND_MAPPING["monitor"]
    monkeypatch.delenv("HF_TOKEN", raising=False)
    a = build_parser("sft").parse_args(["cfg.yaml", "--hub_token", "hf_abc"])
    take_hub_token(a)
    assert os.environ["HF_TOKEN"] == "hf_abc" and not hasattr(a, "hub_token")
    monkeypatch.delenv("HF_TOKEN", raising=False)


def test_nested_orchestrator_schema_is_translated_to_the_flat_keys():
    from surogate_b200.grpo.config import OrchestratorConfig
    from surogate_b200.grpo.config_compat import flatten_orchestrator_config, is_nested_schema, temperature_at

    flat_in = {"model": "m", "group_size": 4, "environment": "markdown-table-qa"}
    assert not is_nested_schema(flat_in) and flatten_orchestrator_config(flat_in) == (flat_in, [])
    nested = {
        "model": {"name": "Qwen/Qwen3-4B", "lora_adapter": "policy"},
        "client": {"base_url": ["http://a:8000/v1", "http://b:8000/v1"], "timeout": 900, "api_key_var": "MYKEY", "headers": {"X-A": "1"}, "skip_model_check": True},
        "sampling": {"temp_scheduler": {"type": "cosine", "start_temperature": 1.2, "end_temperature": 0.6, "total_steps": 100}, "top_p": 0.95, "max_tokens": 768,
                     "repetition_penalty": 1.1, "min_tokens": 0, "extra_body": {"top_k": 50}},
        "env": [{"id": "multihop-tools", "args": {"hops": 2}}, {"id": "other"}],
        "batch_size": 64, "rollouts_per_example": 8, "sequence_len": 4096, "max_steps": 300, "max_off_policy_steps": 6, "max_async_level": 1, "seed": 7,
        "max_inflight_rollouts": 256, "output_dir": "outputs/run1",
        "buffer": {"easy_threshold": 1.0, "hard_threshold": 0.0, "online_difficulty_filtering": True, "normal_pool_min_examples": 100, "hash_keys": ["task", "prompt"]},
        "rollout_depth": {"enabled": True, "quantile": 0.8, "min_depth": 2, "max_depth": 16, "probe_interval": 8, "ema": 0.3},
        "advantage": {"type": "custom", "import_path": "my_pkg.adv.compute", "kwargs": {"a": 1}},
        "filters": [{"type": "gibberish", "token_id_threshold": 100000, "logprob_offset": 2.0}, {"type": "repetition", "window": 3000, "prob_threshold": 0.99, "enforce": True}],
        "ckpt": {"interval": 25, "keep_last": 3}, "eval": {"interval": 50, "rollouts_per_example": 2, "num_examples": 32},
        "weight_broadcast": {"type": "nccl", "port": 29501}, "rollout_transport": {"type": "zmq", "host": "10.0.0.1", "port": 5566},
        "ruler": {"enabled": True, "judge_model": "j"}, "tasks_per_minute": 10.0, "dump_metrics": True, "val": {"interval": 5, "num_examples": 8}, "strict_async_level": True,
    }
    flat, notes = flatten_orchestrator_config(nested)
    assert flat["scheduler"] == "async" and flat["model"] == "Qwen/Qwen3-4B" and flat["served_model"] == "policy"
    assert flat["base_url"] == "http://a:8000/v1" and len(flat["base_urls"]) == 2 and flat["request_timeout_s"] == 900.0 and flat["api_key_var"] == "MYKEY"
    assert flat["temperature_schedule"] == {"type": "cosine", "start": 1.2, "end": 0.6, "total_steps": 100} and flat["top_p"] == 0.95 and flat["max_tokens"] == 768
    assert flat["extra_sampling"] == {"top_k": 50, "repetition_penalty": 1.1}
    assert flat["environment"] == "multihop-tools" and flat["environment_args"] == {"hops": 2}
    assert flat["group_size"] == 8 and flat["batch_size"] == 64 and flat["prompts_per_step"] == 8 and flat["max_inflight"] == 32 and flat["rows_per_step"] == 0
    assert flat["buffer"] == {"easy_threshold": 1.0, "hard_threshold": 0.0, "online_difficulty_filtering": True, "min_normal": 100}
    assert flat["depth"] == {"enabled": True, "quantile": 0.8, "min_cap": 2, "max_cap": 16, "probe_every": 8}
    assert flat["advantage"] == "my_pkg.adv:compute" and flat["filters"][0]["enforce"] is False and flat["filters"][1]["enforce"] is True
    assert flat["checkpoint_every"] == 25 and flat["keep_checkpoints"] == 3 and flat["checkpoint_dir"] == os.path.join("outputs/run1", "orch_checkpoints")
    assert flat["eval_every"] == 50 and flat["eval_samples"] == 2 and flat["eval_examples"] == 32
    assert flat["weight_broadcast"] == "nccl" and flat["transport"] == "zmq" and flat["zmq_endpoint"] == "tcp://10.0.0.1:5566"
    assert flat["weight_dir"] == os.path.join("outputs/run1", "weights") and flat["transport_dir"] == os.path.join("outputs/run1", "rollouts")
    text = "\n".join(notes)
    assert [e["id"] for e in flat["environments"]] == ["multihop-tools", "other"] and "ruler" not in text and flat["ruler"]["judge_model"] == "j" and "strict_async_level" in text and "tasks_per_minute" not in text and flat["tasks_per_minute"] == 10.0
    assert flat["metrics_file"].endswith("orchestrator_metrics.jsonl") and (flat["val_every"], flat["val_examples"], flat["val_samples"]) == (5, 8, 1) and "skip_model_check" not in text
    # the flat result is a valid orchestrator config of this package
    from surogate_b200.config.loader import coerce_fields

    cfg = OrchestratorConfig(**coerce_fields(OrchestratorConfig, {k: v for k, v in flat.items() if k in OrchestratorConfig.__dataclass_fields__}))
    assert cfg.group_size == 8 and cfg.transport == "zmq" and cfg.extra_sampling["top_k"] == 50
    with pytest.raises(ValueError):
        flatten_orchestrator_config({"sampling": {"temperature": 1.0, "temp_scheduler": {"start_temperature": 1.0, "end_temperature": 0.5}}})
    sch = flat["temperature_schedule"]
    assert temperature_at(0, sch, 300) == 1.2 and abs(temperature_at(50, sch, 300) - 0.9) < 1e-9 and temperature_at(100, sch, 300) == temperature_at(500, sch, 300) == 0.6
    assert abs(temperature_at(5, {"type": "linear", "start": 1.0, "end": 0.0, "total_steps": None}, 10) - 0.5) < 1e-12


def test_per_token_filter_rules_and_enforce_flag():
    from surogate_b200.grpo.orchestration.filters import apply_filters, make_filters
    from surogate_b200.grpo.packer import Rollout
    import math

    V = 1000
    thr = -math.log(V) - 2.0
    ok = Rollout([1], [5, 999, 7], [-0.1, thr + 0.1, -0.2], 0.0, 1.0, 0, 0, {})
    rare = Rollout([1], [5, 999, 7], [-0.1, thr - 0.1, -0.2], 0.0, 1.0, 0, 0, {})           # a rare id sampled below the threshold
    common = Rollout([1], [5, 100, 7], [-0.1, thr - 0.1, -0.2], 0.0, 1.0, 0, 0, {})        # same surprise on a common id: fine
    loop = Rollout([1], list(range(10)), [-0.001] * 10, 0.0, 1.0, 0, 0, {})                 # ten near-certain tokens in a row
    brk = Rollout([1], list(range(10)), [-0.001] * 4 + [-1.0] + [-0.001] * 5, 0.0, 1.0, 0, 0, {})
    fs = make_filters([{"type": "gibberish", "token_id_threshold": 500, "logprob_offset": 2.0, "enforce": False}, {"type": "repetition", "window": 6, "prob_threshold": 0.99}], V)
    rs = [ok, rare, common, loop, brk]
    for r in rs:
        r.completion_mask = [1] * len(r.completion_ids)
    stats = apply_filters(fs, rs)
    assert stats == {"filter/gibberish": 0.2, "filter/repetition": 0.2}
    assert rare.meta["filtered"] == "gibberish" and sum(rare.completion_mask) == 3           # counted only: enforce is off
    assert loop.meta["filtered"] == "repetition" and sum(loop.completion_mask) == 0          # enforced: leaves the loss
    assert "filtered" not in ok.meta and "filtered" not in common.meta and "filtered" not in brk.meta


def test_inference_config_takes_the_short_keys_and_builds_the_engine_command(monkeypatch):
    from surogate_b200.grpo.config import InferenceConfig
    from surogate_b200.grpo.inference import server_command

    monkeypatch.delenv("SUROGATE_ENGINE_MEMORY_FRACTION", raising=False)
    cfg = InferenceConfig(model="m", tp=2, dp=2, max_lora_rank=24, weight_broadcast_type="nccl", kv_cache_dtype="fp8", max_num_seqs=256, enforce_eager=True,
                          enable_auto_tool_choice=True, reasoning_parser="qwen3", enable_prefix_caching=False, seed=3, dtype="bfloat16", enable_expert_parallel=True,
                          rope_scaling={"rope_type": "yarn", "factor": 2.0}, api_server_count=4)
    assert (cfg.tensor_parallel_size, cfg.data_parallel_size, cfg.max_lora_rank, cfg.weight_broadcast, cfg.api_server_count) == (2, 2, 32, "nccl", 1)
    cmd = server_command(cfg)
    text = " ".join(cmd)
    for part in ("--tensor-parallel-size 2", "--data-parallel-size 2", "--kv-cache-dtype fp8", "--max-num-seqs 256", "--enforce-eager", "--enable-auto-tool-choice --tool-call-parser hermes",
                 "--reasoning-parser qwen3", "--no-enable-prefix-caching", "--seed 3", "--dtype bfloat16", "--enable-expert-parallel", "--enable-lora --max-loras 8 --max-cpu-loras 100 --max-lora-rank 32",
                 "--worker-extension-cls"):
        assert part in text, part
    assert json.loads(cmd[cmd.index("--rope-scaling") + 1]) == {"rope_type": "yarn", "factor": 2.0} and "--api-server-count" not in cmd
    assert InferenceConfig(model="m", enable_lora=False, dp=4).api_server_count == 4
    plain = " ".join(server_command(InferenceConfig(model="m")))
    assert "--kv-cache-dtype" not in plain and "--dtype" not in plain and "--seed" not in plain and "prefix-caching" not in plain
    with pytest.raises(ValueError):
        InferenceConfig(model="m", max_lora_rank=1024)
    with pytest.raises(ValueError):
        InferenceConfig(model="m", weight_broadcast="carrier-pigeon")


def test_reporter_keys_and_enable_thinking_field(monkeypatch):
    import sys
    import types

    from surogate_b200.config.sft_config import DatasetConfig, SFTConfig
    from surogate_b200.data.datasets import preprocess_preference
    from surogate_b200.train.reporter import make_reporters

    cfg = SFTConfig.from_dict(dict(model=json.dumps(_tiny_model()), synthetic_data=True, wandb_project="P", wandb_name="N", aim_experiment="E", aim_repo="/r", aim_name="A"))
    seen = {}
    wandb = types.ModuleType("wandb")
    wandb.init = lambda **kw: seen.setdefault("wandb", kw) and types.SimpleNamespace(finish=lambda: None)
    aim = types.ModuleType("aim")

    class Run(dict):
        def __init__(self, **kw):
            seen["aim"] = kw

        def track(self, *a, **k):
            pass

        def close(self):
            pass

    aim.Run = Run
    monkeypatch.setitem(sys.modules, "wandb", wandb)
    monkeypatch.setitem(sys.modules, "aim", aim)
    reps = make_reporters(["wandb", "aim"], "run-1", config=json.loads(cfg.to_json()))
    assert seen["wandb"]["project"] == "P" and seen["wandb"]["name"] == "N" and seen["aim"] == {"experiment": "E", "repo": "/r"} and reps[1].run.name == "A"
    seen.clear()
    make_reporters(["wandb", "aim"], "run-1", config={})
    assert seen["wandb"]["project"] == "Surogate" and seen["wandb"]["name"] == "run-1" and seen["aim"] == {"experiment": "Surogate"}

    row = {"prompt": "q", "chosen": "a", "rejected": "b", "enable_thinking": False, "think": "true"}
    assert preprocess_preference(DatasetConfig(type="preference"), row)["enable_thinking"] is False
    assert preprocess_preference(DatasetConfig(type="preference", enable_thinking_field="think"), row)["enable_thinking"] is True
    assert "enable_thinking" not in preprocess_preference(DatasetConfig(type="preference"), {"prompt": "q", "chosen": "a", "rejected": "b"})
    with pytest.raises(ValueError, match="enable-thinking field"):
        preprocess_preference(DatasetConfig(type="preference", enable_thinking_field="nope"), row)

    class Tok:
        eos_token_id, pad_token_id = 1, 0

        def apply_chat_template(self, msgs, add_generation_prompt=False, enable_thinking=None):
            seen["thinking"] = enable_thinking
            return "p"

        def encode(self, text):
            return [5, 6] if text == "p" else [7]

    from surogate_b200.dpo.data import encode_pair

    encode_pair(Tok(), {"prompt": [{"role": "user", "content": "q"}], "chosen": "a", "rejected": "b", "enable_thinking": False}, 8, 4)
    assert seen["thinking"] is False


def test_export_carries_the_tokenizer_files(tmp_path):
    from surogate_b200.io.hf_checkpoint import copy_tokenizer_files
    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    src = tmp_path / "src"
    os.makedirs(src)
    for fn in ("tokenizer.json", "tokenizer_config.json", "generation_config.json", "unrelated.txt"):
        (src / fn).write_text(fn)
    tr = Trainer(TrainerConfig(model=_tiny_model(), batch_size=1, seq_len=8, backend="torch", recipe="bf16", optimizer="adamw"), device=torch.device("cpu"))
    tr.init_weights(0)
    tr.tokenizer_source = str(src)
    out = tmp_path / "out"
    tr.export_model(str(out))
    assert sorted(os.listdir(out)) == ["config.json", "generation_config.json", "model.safetensors", "tokenizer.json", "tokenizer_config.json"]
    (out / "tokenizer.json").write_text("kept")
    assert copy_tokenizer_files(str(src), str(out)) == [] and (out / "tokenizer.json").read_text() == "kept"
    assert copy_tokenizer_files(None, str(out)) == [] and copy_tokenizer_files(str(out), str(out)) == []


def test_debug_commands_take_a_training_config(tmp_path, capsys):
    """``surogate debug <sub> config.yaml --output report.jsonl``: model, sequence length and micro-batch come from the config; the
    tracing commands build the model as the run would (LoRA), gradients can be followed over several updates."""
    from surogate_b200.cli import debug as cli
    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    model = dict(_tiny_model(), n_layers=2)
    tr = Trainer(TrainerConfig(model=model, batch_size=1, seq_len=16, backend="torch", recipe="bf16", optimizer="adamw"), device=torch.device("cpu"))
    tr.init_weights(0)
    base = str(tmp_path / "base")
    tr.export_model(base, model)
    cfg = tmp_path / "cfg.yaml"
    cfg.write_text(yaml.safe_dump(dict(model=base, sequence_len=24, per_device_train_batch_size=2, lora=True, lora_rank=4, lora_alpha=8, recipe="bf16", optimizer="adamw",
                                       datasets=[{"path": "x.jsonl"}])))
    target = cli.resolve_target(str(cfg))
    assert target[0] == base and target[1:3] == (24, 2) and target[3].lora and cli.resolve_target(base) == (base, 128, 1, None)
    assert cli.resolve_target(str(cfg), seq_len=8, batch=1)[1:3] == (8, 1)
    out = tmp_path / "grads.jsonl"
    assert cli.main(["gradients", str(cfg), "--output", str(out), "--steps", "2", "--seq-len", "12"]) == 0
    rows = [json.loads(l) for l in open(out)]
    assert {r["step"] for r in rows} == {0, 1} and all("lora" in r["param"].lower() for r in rows) and all(r["absmax"] == r["absmax"] for r in rows)
    assert cli.main(["activations", str(cfg), "--output", str(tmp_path / "acts.jsonl")]) == 0
    assert cli.main(["weights", str(cfg)]) == 0 and cli.main(["tensor-arena", str(cfg), "--output", str(tmp_path / "arena.jsonl")]) == 0
    capsys.readouterr()
    assert os.path.getsize(tmp_path / "acts.jsonl") > 0 and os.path.getsize(tmp_path / "arena.jsonl") > 0


def test_push_to_hub_creates_the_repository_and_uploads_the_directory(tmp_path):
    from surogate_b200.hub import HubError, push_to_hub

    calls = []

    class Api:
        def create_repo(self, repo_id, **kw):
            calls.append(("create", repo_id, kw))

        def upload_folder(self, **kw):
            calls.append(("upload", kw))
            return "commit-url"

    out = tmp_path / "model"
    os.makedirs(out)
    (out / "config.json").write_text("{}")
    assert push_to_hub("me/my-model", str(out), private=True, revision="master", token="t", api=Api()) == "commit-url"
    assert calls[0] == ("create", "me/my-model", {"token": "t", "private": True, "exist_ok": True})
    up = calls[1][1]
    assert up["repo_id"] == "me/my-model" and up["revision"] == "main" and up["folder_path"] == str(out) and "step_*" in up["ignore_patterns"] and up["commit_message"] == "Upload model"
    with pytest.raises(HubError, match="not a directory"):
        push_to_hub("me/x", str(tmp_path / "missing"), api=Api())

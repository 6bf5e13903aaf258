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

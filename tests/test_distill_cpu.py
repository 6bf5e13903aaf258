"""KD sidecars: format round trip, capture from a teacher held by the Trainer, training with the distillation term."""
import json
import os

import numpy as np
import pytest
import torch

from surogate_b200.data.loader import write_synthetic_tokens
from surogate_b200.distill.capture import capture_shard, native_teacher
from surogate_b200.distill.sidecar import KD_MAGIC, SidecarReader, SidecarWriter
from surogate_b200.runtime.trainer import Trainer, TrainerConfig

MODEL = dict(architecture="Qwen3ForCausalLM", vocab_size=96, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64,
             tie_word_embeddings=True)


def _trainer(seed):
    t = Trainer(TrainerConfig(model=MODEL, batch_size=2, seq_len=16, recipe="bf16", optimizer="adamw", learning_rate=2e-2, zero_level=0),
                device=torch.device("cpu"))
    t.init_weights(seed=seed)
    return t


def test_sidecar_round_trip(tmp_path):
    p = os.path.join(tmp_path, "a.kd")
    w = SidecarWriter(p, top_k=4, vocab_size=96, temperature=2.0)
    idx = np.arange(40, dtype=np.int32).reshape(10, 4)
    lp = -np.linspace(0.1, 4.0, 40, dtype=np.float32).reshape(10, 4)
    w.add(idx, lp)
    assert w.close() == 10
    with open(p, "rb") as f:
        assert f.read(8) == KD_MAGIC
    r = SidecarReader(p)
    assert (r.K, r.N, r.vocab, r.temperature) == (4, 10, 96, 2.0)
    i2, l2 = r.rows(3, 5)
    assert np.array_equal(i2, idx[3:8]) and np.allclose(l2, lp[3:8], atol=2e-3)


def test_capture_and_distill(tmp_path):
    shard = write_synthetic_tokens(os.path.join(tmp_path, "train-000.bin"), 4, 16, 96, seed=1)
    teacher, student = _trainer(11), _trainer(22)
    kd_path = capture_shard(shard, native_teacher(teacher), 16, top_k=8, vocab=96, rows_per_call=2)
    r = SidecarReader(kd_path)
    assert r.N == 64 and r.K == 8
    from surogate_b200.data.tokfile import read_token_file

    tok, _, _, _ = read_token_file(shard)
    x = np.asarray(tok[:32]).reshape(2, 16)
    # the sidecar holds the teacher's own top-K log-probs
    lg = teacher.logits(x)
    lp = torch.log_softmax(lg, -1).topk(8, -1)
    i0, l0 = r.rows(0, 32)
    assert np.array_equal(i0.reshape(2, 16, 8), lp.indices.numpy()) and np.allclose(l0.reshape(2, 16, 8), lp.values.numpy(), atol=5e-3)
    y = np.concatenate([x[:, 1:], np.full((2, 1), -100, np.int32)], axis=1)
    kd = {"idx": torch.from_numpy(i0.reshape(2, 16, 8)), "logp": torch.from_numpy(l0.reshape(2, 16, 8)), "weight": 1.0, "ce_weight": 0.0}
    first = last = None
    for _ in range(25):
        res = student.forward_backward(x, y, kd=kd)
        student.optimizer_step()
        v = float(res["loss_sum"] / res["n_valid"])
        first = v if first is None else first
        last = v
    assert last < 0.5 * first, (first, last)  # the student moves toward the teacher's distribution


def test_api_teacher_against_a_local_openai_style_server(tmp_path):
    """``prompt_logprobs`` of an OpenAI-compatible completions endpoint (what vLLM serves) captured into a sidecar: concurrent rows,
    one injected failure retried, alignment (entry t predicts token t -> stored at t-1), resume skips a complete sidecar."""
    import json
    import threading
    from http.server import BaseHTTPRequestHandler, HTTPServer

    from surogate_b200.distill.capture import api_teacher_rows, capture, sidecar_complete

    teacher = _trainer(5)
    calls = {"n": 0, "failed": False}
    lock = threading.Lock()

    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            with lock:
                calls["n"] += 1
                fail = not calls["failed"]
                calls["failed"] = True
            if fail:
                self.send_response(503)
                self.end_headers()
                return
            row = np.asarray(body["prompt"], np.int32)[None]
            with lock:
                lp = torch.log_softmax(teacher.logits(row)[0], -1)
            k = body["prompt_logprobs"]
            out = [None]
            for t in range(1, row.shape[1]):
                top = lp[t - 1].topk(k)
                out.append({str(int(i)): {"logprob": float(v)} for i, v in zip(top.indices, top.values)})
            data = json.dumps({"choices": [{"prompt_logprobs": out}]}).encode()
            self.send_response(200)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

    srv = HTTPServer(("127.0.0.1", 0), H)
    th = threading.Thread(target=srv.serve_forever, daemon=True)
    th.start()
    try:
        shard = write_synthetic_tokens(os.path.join(tmp_path, "train-000.bin"), 4, 16, 96, seed=2)
        direct = api_teacher_rows(f"http://127.0.0.1:{srv.server_port}/v1", "teacher", 4, workers=3, timeout_s=20)
        (kd_path,) = capture([shard], None, 16, 4, 96, rows_per_call=4, direct=direct)
        n_first = calls["n"]
        assert n_first == 5 and sidecar_complete(shard, 16, 4)            # 4 rows + the retried one
        assert capture([shard], None, 16, 4, 96, rows_per_call=4, direct=direct) == [kd_path] and calls["n"] == n_first     # resumed: no request
    finally:
        srv.shutdown()
    from surogate_b200.data.tokfile import read_token_file

    tok, _, _, _ = read_token_file(shard)
    x = np.asarray(tok[:16]).reshape(1, 16)
    want = torch.log_softmax(teacher.logits(x)[0], -1).topk(4)
    i0, l0 = SidecarReader(kd_path).rows(0, 16)
    assert np.array_equal(i0[:15], want.indices.numpy()[:15]) and np.allclose(l0[:15], want.values.numpy()[:15], atol=5e-3)
    assert np.all(l0[15] == -30.0)          # nothing predicts past the last token of a row


def test_distillation_section_spellings_and_sidecar_directory(tmp_path, monkeypatch):
    """The ``distillation`` section accepts both spellings of its keys, is on when present, validates K and temperature; sidecars
    captured into ``kd_dir`` are the ones a training run with the same section reads."""
    from surogate_b200.config.sft_config import DistillationConfig, SFTConfig
    from surogate_b200.distill.capture import capture
    from surogate_b200.distill.sidecar import sidecar_path

    d = DistillationConfig(teacher_model="T", kd_dir="/x", kd_weight=0.3)
    assert d.enabled and d.teacher == "T" and d.sidecar_dir == "/x" and abs(d.ce_weight - 0.7) < 1e-12 and d.top_k == 32
    assert DistillationConfig(kd_weight=0.5, ce_weight=1.0).ce_weight == 1.0 and not DistillationConfig(enabled=False).enabled
    monkeypatch.setenv("MY_KEY", "secret")
    assert DistillationConfig(teacher_api_key_var="MY_KEY").api_key() == "secret" and DistillationConfig(teacher_api_key_var="UNSET_VAR_X").api_key() == "EMPTY"
    for bad in (dict(top_k=0), dict(top_k=2000), dict(temperature=0.0)):
        with pytest.raises(ValueError, match="E115"):
            DistillationConfig(**bad)

    model = dict(architecture="Qwen3ForCausalLM", vocab_size=96, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64, tie_word_embeddings=True)
    kd_dir = str(tmp_path / "kd")
    base = dict(model=json.dumps(model), synthetic_data=True, sequence_len=16, per_device_train_batch_size=2, gradient_accumulation_steps=1, max_steps=2, lora=False,
                optimizer="adamw", learning_rate=1e-2, save_steps=0, eval_steps=0, recipe="bf16", zero_level=0, from_scratch=True, output_dir=str(tmp_path / "run"),
                distillation=dict(teacher_model="unused", top_k=4, kd_weight=1.0, kd_dir=kd_dir))
    cfg = SFTConfig.from_dict(base)
    assert cfg.distillation.enabled and cfg.distillation.sidecar_dir == kd_dir
    from surogate_b200.train.sft import prepare_data, resolve_model_config, run_training

    shards = prepare_data(cfg, resolve_model_config(cfg), rank=0)["train"]
    teacher = _trainer(3)
    out = capture(shards, native_teacher(teacher), 16, 4, 96, out_dir=kd_dir)
    assert [os.path.dirname(p) for p in out] == [kd_dir] * len(shards) and not os.path.exists(sidecar_path(shards[0]))
    assert capture(shards, None, 16, 4, 96, out_dir=kd_dir) == out  # complete sidecars are kept: no teacher is called
    r = run_training(cfg)
    assert r["steps"] == 2 and np.isfinite(r["final"]["loss"])


def test_distill_capture_command_reads_the_config(tmp_path, monkeypatch, capsys):
    """``surogate distill-capture config.yaml`` tokenises like the run will, takes teacher / K / directory from the section and
    writes one sidecar per shard."""
    import yaml

    from surogate_b200.cli import distill as cli
    from surogate_b200.distill import capture as cap

    model = dict(architecture="Qwen3ForCausalLM", vocab_size=96, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64, tie_word_embeddings=True)
    cfg = dict(model=json.dumps(model), synthetic_data=True, sequence_len=16, per_device_train_batch_size=2, output_dir=str(tmp_path / "run"), lora=False,
               distillation=dict(teacher_model="my-teacher", top_k=4, temperature=2.0, teacher_batch_size=3, kd_dir=str(tmp_path / "kd")))
    path = tmp_path / "cfg.yaml"
    path.write_text(yaml.safe_dump(cfg))
    seen = {}
    teacher = _trainer(3)

    def fake_hf_teacher(name, device):
        seen.update(name=name, device=device)
        return native_teacher(teacher)

    monkeypatch.setattr(cap, "hf_teacher", fake_hf_teacher)
    assert cli.main([str(path), "--device", "cpu"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["sidecars"]
    assert seen == {"name": "my-teacher", "device": "cpu"} and out and all(p.startswith(str(tmp_path / "kd")) for p in out)
    r = SidecarReader(out[0])
    assert r.K == 4 and abs(r.temperature - 2.0) < 1e-6
    with pytest.raises(SystemExit):
        cli.main([])

"""Named tensors written to files during a run, switched on by environment variables (``surogate_b200/debug/dump.py``)."""
import json
import os

import numpy as np
import torch

from surogate_b200.debug.dump import env_dump_hook, load_dump, parse_names, qualified, sanitise
from surogate_b200.runtime.trainer import Trainer, TrainerConfig

HF = dict(architectures=["Qwen3ForCausalLM"], vocab_size=96, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
          head_dim=16, rms_norm_eps=1e-6, tie_word_embeddings=True, rope_theta=10000.0, max_position_embeddings=128)


def test_names_and_file_names():
    everything, wanted = parse_names("blocks[3].ln1, d_blocks[2].d_x ,loss,all")
    assert everything and wanted == {(3, "ln1"), (2, "d_x"), (None, "loss")}
    assert sanitise("blocks[3].ln1") == "blocks_3_.ln1" and qualified("ln1", 3) == "blocks[3].ln1" and qualified("d_x", 0) == "d_blocks[0].d_x" and qualified("loss", None) == "loss"
    assert env_dump_hook({}) is None and env_dump_hook({"SUROGATE_DEBUG_DUMP_TENSORS": "x"}) is None


def test_a_step_writes_the_named_tensors(tmp_path, monkeypatch):
    def trainer():
        t = Trainer(TrainerConfig(model=HF, batch_size=2, seq_len=16, grad_accum=1, recipe="bf16", optimizer="adamw", param_dtype="fp32", backend="torch", use_cuda_graphs=False),
                    device=torch.device("cpu"))
        t.init_weights(0)
        return t

    x = torch.randint(0, 96, (2, 16))
    y = torch.roll(x, -1, 1)
    # which names a block produces: record them with the programmatic hook first
    seen = []
    t = trainer()
    t.executor.options.dump_tensors = lambda name, layer, val: seen.append((name, layer, tuple(val.shape), val.is_floating_point()))
    t.step(x, y)
    block_names = [n for n, l, _, fp in seen if l == 1 and fp]
    assert block_names
    name = block_names[0]
    shape = next(s for n, l, s, _ in seen if n == name and l == 1)

    monkeypatch.setenv("SUROGATE_DEBUG_DUMP_TENSORS", f"blocks[1].{name}")
    monkeypatch.setenv("SUROGATE_DEBUG_DUMP_DIR", str(tmp_path / "one"))
    t = trainer()
    assert t.executor.options.dump_tensors is not None
    t.step(x, y)
    files = sorted(os.listdir(tmp_path / "one"))
    assert files == [sanitise(f"blocks[1].{name}") + ".bin", sanitise(f"blocks[1].{name}") + ".json"]
    meta = json.load(open(tmp_path / "one" / files[1]))
    assert meta == {"name": f"blocks[1].{name}", "dtype": "float32", "shape": list(shape)}
    arr = load_dump(str(tmp_path / "one"), f"blocks[1].{name}")
    assert arr.shape == shape and np.isfinite(arr).all() and os.path.getsize(tmp_path / "one" / files[0]) == arr.size * 4

    # a bare name dumps every layer; the layer filter narrows it again
    monkeypatch.setenv("SUROGATE_DEBUG_DUMP_TENSORS", name)
    monkeypatch.setenv("SUROGATE_DEBUG_DUMP_DIR", str(tmp_path / "every"))
    trainer().step(x, y)
    assert {f for f in os.listdir(tmp_path / "every") if f.endswith(".bin")} == {sanitise(f"blocks[{l}].{name}") + ".bin" for l in (0, 1)}
    monkeypatch.setenv("SUROGATE_DEBUG_DUMP_LAYER", "0")
    monkeypatch.setenv("SUROGATE_DEBUG_DUMP_DIR", str(tmp_path / "layer0"))
    trainer().step(x, y)
    assert {f for f in os.listdir(tmp_path / "layer0") if f.endswith(".bin")} == {sanitise(f"blocks[0].{name}") + ".bin"}


def test_op_profile_counts_every_dispatched_op(monkeypatch, capsys):
    import io

    monkeypatch.setenv("SUROGATE_OP_PROFILE", "1")
    t = Trainer(TrainerConfig(model=HF, batch_size=2, seq_len=16, grad_accum=1, recipe="bf16", optimizer="adamw", param_dtype="fp32", backend="torch", use_cuda_graphs=True),
                device=torch.device("cpu"))
    t.init_weights(0)
    prof = t.executor.op_profile
    assert prof is not None and not t._graphs_allowed(None, None, None)
    x = torch.randint(0, 96, (2, 16))
    t.step(x, torch.roll(x, -1, 1))
    rows = prof.rows()
    kinds = {r[0] for r in rows}
    assert "fused_lm_head_loss" in kinds and any("rmsnorm" in k for k in kinds) and any("matmul" in k or "linear" in k for k in kinds)
    assert abs(sum(r[4] for r in rows) - 1.0) < 1e-6 and all(r[2] >= 1 and r[1] >= 0 for r in rows) and rows == sorted(rows, key=lambda r: -r[1])
    per_layer = next(r for r in rows if "rmsnorm" in r[0])
    assert per_layer[2] >= 2  # two layers: the kind was dispatched at least once per layer
    buf = io.StringIO()
    prof.report(buf)
    assert "[op-profile]" in buf.getvalue() and "fused_lm_head_loss" in buf.getvalue()
    prof.reset()
    assert prof.rows() == []
    monkeypatch.setenv("SUROGATE_OP_PROFILE", "0")
    t2 = Trainer(TrainerConfig(model=HF, batch_size=2, seq_len=16, grad_accum=1, recipe="bf16", optimizer="adamw", param_dtype="fp32", backend="torch"), device=torch.device("cpu"))
    assert t2.executor.op_profile is None


def test_nonfinite_check_names_the_first_bad_tensor(monkeypatch):
    import pytest

    monkeypatch.setenv("SUROGATE_DEBUG_CHECK_NONFINITE", "1")
    t = Trainer(TrainerConfig(model=HF, batch_size=2, seq_len=16, grad_accum=1, recipe="bf16", optimizer="adamw", param_dtype="fp32", backend="torch", use_cuda_graphs=True),
                device=torch.device("cpu"))
    t.init_weights(0)
    assert t.executor.options.check_finite and not t._graphs_allowed(None, None, None)
    x = torch.randint(0, 96, (2, 16))
    t.step(x, torch.roll(x, -1, 1))  # a healthy step passes
    name, w = next((n, w) for n, w in t.store.named_full_tensors() if "embed" in n)
    w = w.clone().float()
    w[0, :4] = float("nan")
    t.store.load_tensor(name, w)
    t.store.sync_work_from_master()
    with pytest.raises(FloatingPointError, match="non-finite values in"):
        t.step(x * 0, torch.roll(x, -1, 1))  # token 0 reads the poisoned embedding row

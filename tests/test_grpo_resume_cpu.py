"""The GRPO trainer loop saves checkpoints, continues from the latest one (weights, optimizer step, policy version) and honours
``SUROGATE_GRPO_START_STEP`` when there is none."""
import json
import os

import numpy as np
import pytest

from surogate_b200.grpo.config import GRPOConfig
from surogate_b200.grpo.packer import Rollout, pack_rollouts
from surogate_b200.grpo.trainer import run_grpo, start_step_override
from surogate_b200.grpo.transport.filesystem import FilesystemTransport

MODEL = dict(architecture="Qwen3ForCausalLM", vocab_size=96, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64, tie_word_embeddings=True)


def _config(tmp_path, **kw):
    d = dict(model=json.dumps(MODEL), sequence_len=16, per_device_train_batch_size=2, gradient_accumulation_steps=1, max_steps=4, lora=False, optimizer="adamw",
             learning_rate=1e-3, save_steps=2, recipe="bf16", zero_level=0, from_scratch=True, output_dir=str(tmp_path / "run"), transport_dir=str(tmp_path / "rollouts"),
             weight_dir=str(tmp_path / "weights"), log_file=str(tmp_path / "log.json"))
    d.update(kw)
    return GRPOConfig.from_dict(d)


def _send_batches(directory, steps):
    tr = FilesystemTransport(directory)
    rng = np.random.default_rng(0)
    for step in steps:
        rollouts = [Rollout(prompt_ids=list(rng.integers(1, 90, 4)), completion_ids=list(rng.integers(1, 90, 6)), logprobs=list(-rng.random(6)), advantage=float(a), group=i // 2)
                    for i, a in enumerate((1.0, -1.0, 0.5, -0.5))]
        b = pack_rollouts(rollouts, 16, 2)[0]
        tr.send(step, b.arrays(), {"policy_version": step, "reward_mean": 0.0})


def test_start_step_variable(monkeypatch):
    monkeypatch.delenv("SUROGATE_GRPO_START_STEP", raising=False)
    assert start_step_override() is None
    monkeypatch.setenv("SUROGATE_GRPO_START_STEP", "7")
    assert start_step_override() == 7
    for bad in ("x", "-1"):
        monkeypatch.setenv("SUROGATE_GRPO_START_STEP", bad)
        with pytest.raises(ValueError, match="SUROGATE_GRPO_START_STEP"):
            start_step_override()


def test_checkpoint_then_continue(tmp_path, monkeypatch):
    monkeypatch.delenv("SUROGATE_GRPO_START_STEP", raising=False)
    _send_batches(str(tmp_path / "rollouts"), range(4))
    first = run_grpo(_config(tmp_path, max_steps=3))
    assert first["steps"] == 3
    ckpts = sorted(d for d in os.listdir(tmp_path / "run") if d.startswith("step_"))
    assert ckpts == ["step_00000002"]
    versions = sorted(os.listdir(tmp_path / "weights"))
    # a second process with the same directories: continues after step 2 at policy version 2, runs steps 2 and 3 only
    second = run_grpo(_config(tmp_path, max_steps=4))
    assert second["steps"] == 2
    assert [h["off_policy"] for h in second["history"]] == [0, 0]  # batches of versions 2 and 3 met a trainer at versions 2 and 3
    assert "v000004" in os.listdir(tmp_path / "weights") and sorted(os.listdir(tmp_path / "weights")) != versions
    assert "continuing at step 2, policy version 2" in open(tmp_path / "log.json").read()
    # no checkpoint + the variable: the loop starts at that step
    monkeypatch.setenv("SUROGATE_GRPO_START_STEP", "3")
    third = run_grpo(_config(tmp_path, max_steps=4, output_dir=str(tmp_path / "fresh"), weight_dir=str(tmp_path / "w2")))
    assert third["steps"] == 1 and any("3" in v for v in os.listdir(tmp_path / "w2"))
    # resume switched off: from step 0 whatever the directory holds
    monkeypatch.delenv("SUROGATE_GRPO_START_STEP")
    assert run_grpo(_config(tmp_path, max_steps=1, resume_from_checkpoint=False, save_steps=0))["steps"] == 1

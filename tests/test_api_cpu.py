"""The trainer-level API under the reference's names (``surogate_b200/api.py``): micro-steps + update equal the engine's own step,
custom per-token gradients and distillation micro-steps, config objects, the loader writing into caller-owned arrays."""
import json
import os

import numpy as np
import pytest
import torch

from surogate_b200.api import DataLoader, LoRAAdapterConfig, OptimizerConfig, PretrainedConfig, QLoRAConfig, RuntimeOptions, SurogateTrainer, SystemInfo
from surogate_b200.data.loader import write_synthetic_tokens

HF = dict(architectures=["Qwen3ForCausalLM"], vocab_size=96, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
          head_dim=16, rms_norm_eps=1e-6, tie_word_embeddings=True, rope_theta=10000.0, max_position_embeddings=128)


def _trainer(grad_accum=2, **kw):
    cfg = PretrainedConfig.from_hf_dict(HF, "fp32")
    t = SurogateTrainer(1, cfg, RuntimeOptions(recipe="bf16", use_cuda_graphs=False), batch_size=2, seq_len=16, grad_accum=grad_accum, device=torch.device("cpu"),
                        backend="torch", optimizer="adamw", **kw)
    t.init_weights()
    return t


def test_config_objects():
    o = OptimizerConfig.normuon(lr=0.01, weight_decay=0.0)
    assert o.type == "normuon" and o.normuon_lr == 0.01 and o.learning_rate == 0.01 and OptimizerConfig.adamw_8bit().optimizer == "adamw_8bit"
    o.type = "adamw"
    assert o.optimizer == "adamw" and OptimizerConfig().weight_decay == 0.1
    c = PretrainedConfig.from_hf_dict(dict(HF, attention_bias=True), "bfloat16")
    assert c.head_size == 16 and c.qkv_channels == 16 * 4 and c.dtype == "bf16" and c.use_qkv_bias and c.model_name == "Qwen3ForCausalLM"
    back = c.to_hf_dict()
    assert back["head_dim"] == 16 and back["attention_bias"] is True and back["architectures"] == ["Qwen3ForCausalLM"] and back["vocab_size"] == 96
    assert PretrainedConfig(architecture="qwen2", hidden_size=8, intermediate_size=16, num_attention_heads=2, num_key_value_heads=1, num_hidden_layers=1).to_hf_dict()["architectures"] == ["Qwen2ForCausalLM"]
    r = RuntimeOptions(recipe="fp8-hybrid", shard_weights=True, recompute_att=True, offload_grads=True)
    kw = r.trainer_kwargs()
    assert r.fp8_enabled and not r.fp4_enabled and kw["recipe"] == "fp8_hybrid" and kw["zero_level"] == 3 and kw["recompute"] and kw["offload_grads"]
    r.set_recipe("nvfp4")
    assert r.fp4_enabled and r.recipe_name == "nvfp4" and RuntimeOptions(shard_gradients=True).trainer_kwargs()["zero_level"] == 2
    l = LoRAAdapterConfig(rank=16, alpha=32.0, use_rslora=True)
    assert l.scaling == 8.0 and l.applies_to("model.layers.0.self_attn.q_proj") and not l.applies_to("mlp.up_proj") and l.as_dict()["targets"] == ["q_proj", "k_proj", "v_proj", "o_proj"]
    q = QLoRAConfig(enabled=True, strategy="nvfp4", num_experts=8)
    assert q.is_fp4 and q.is_quantized and q.is_moe and not QLoRAConfig(strategy="fp8").is_quantized
    assert SystemInfo.get_cuda_runtime_version() >= 0 and isinstance(SystemInfo.get_gpu_info(), list) and SystemInfo.get_nccl_version() >= 0
    with pytest.raises(ValueError, match="torchrun"):
        SurogateTrainer(4, c, RuntimeOptions(), 2, 16, 1, device=torch.device("cpu"), backend="torch")


def test_micro_steps_then_update_equal_the_engine_step():
    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    rng = np.random.default_rng(0)
    x = rng.integers(0, 96, (4, 16)).astype(np.int32)
    y = np.roll(x, -1, 1).astype(np.int32)
    y[:, -1] = -100
    t = _trainer()
    assert t.options_without_effect == [] and (t.batch_size, t.seq_length, t.world_size) == (2, 16, 1)
    ref = Trainer(TrainerConfig(model=PretrainedConfig.from_hf_dict(HF, "fp32").to_hf_dict(), batch_size=2, seq_len=16, grad_accum=2, recipe="bf16", optimizer="adamw",
                                param_dtype="fp32", backend="torch", weight_decay=0.1, learning_rate=1e-2, max_grad_norm=0.0, use_cuda_graphs=False), device=torch.device("cpu"))
    ref.init_weights(0)
    opt = OptimizerConfig.adamw(lr=1e-2)
    with pytest.raises(RuntimeError, match="grad_accum is 2"):
        t.update_with_config(opt, 1)
    for step in range(3):
        t.step(x[:2], y[:2])
        t.step(x[2:], y[2:])
        out = t.update_with_config(opt, step + 1)
        want = ref.step(x, y, lr=1e-2)
        assert abs(out["loss"] - want["loss"]) < 1e-5 and abs(out["norm"] - want["norm"]) < 1e-4
    with pytest.raises(RuntimeError, match="queued already"):
        for _ in range(3):
            t.step(x[:2], y[:2])
    t._queue.clear()
    v = t.validate(x[:2], y[:2])
    assert abs(v - ref.validate(x[:2], y[:2])["loss"]) < 1e-5
    lp = t.compute_logprobs(x[:2], y[:2])
    assert lp.shape == (2, 16) and (lp[:, -1] == 0).all() and (lp[:, :-1] < 0).all()
    out = t.train_step_graphed(x, y, opt, 4)
    assert np.isfinite(out["loss"]) and "category.weights" in t.get_allocator_info() or t.get_allocator_info()


def test_custom_loss_and_kd_micro_steps(tmp_path):
    rng = np.random.default_rng(1)
    x = rng.integers(0, 96, (2, 16)).astype(np.int32)
    y = np.roll(x, -1, 1).astype(np.int32)
    y[:, -1] = -100
    t = _trainer(grad_accum=1)
    before = t.compute_logprobs(x, y)
    w = np.where(np.arange(2)[:, None] == 0, 0.05, -0.05).astype(np.float32) * (y != -100)
    for step in range(3):
        t.step_with_custom_loss(x, y, w)
        t.update_with_config(OptimizerConfig.adamw(lr=5e-2, weight_decay=0.0), step + 1)
    after = t.compute_logprobs(x, y)
    assert after[0].sum() > before[0].sum() and after[1].sum() < before[1].sum()      # positive multipliers raise, negative lower the likelihood
    k = 4
    kd_ids = rng.integers(0, 96, (2, 16, k)).astype(np.int32)
    kd_lp = np.log(np.full((2, 16, k), 0.25, np.float32))
    t.step_with_kd(x, y, kd_ids, kd_lp, top_k=k, kd_weight=1.0, ce_weight=0.0)
    out = t.update_with_config(OptimizerConfig.adamw(lr=1e-3), 4)
    assert np.isfinite(out["loss"]) and t.get_kd_loss() == out["loss"] and t.get_kd_loss() == 0.0
    t.save_checkpoint(str(tmp_path / "ck"), 4)
    t.export_model(str(tmp_path / "model"))
    assert os.path.exists(tmp_path / "model" / "config.json") and json.load(open(tmp_path / "model" / "config.json"))["head_dim"] == 16
    t2 = _trainer(grad_accum=1)
    t2.load_checkpoint(str(tmp_path / "ck"), 4)
    assert np.allclose(t2.compute_logprobs(x, y), t.compute_logprobs(x, y), atol=1e-6)
    t3 = SurogateTrainer.from_pretrained(str(tmp_path / "model"), 1, "fp32", RuntimeOptions(use_cuda_graphs=False), 2, 16, 1, device=torch.device("cpu"), backend="torch",
                                         optimizer="adamw")
    assert np.allclose(t3.compute_logprobs(x, y), t.compute_logprobs(x, y), atol=2e-2)   # the export is bf16


def test_loader_fills_caller_arrays(tmp_path):
    shard = write_synthetic_tokens(str(tmp_path / "train-000.bin"), 8, 16, 96, seed=3)
    dl = DataLoader([shard], chunk_size=2 * 16, seed=5)
    assert (dl.num_files, dl.num_tokens, dl.num_chunks, dl.vocab_size, dl.seed, dl.epoch, dl.seq_len) == (1, 128, 4, 96, 5, 0, 0) and dl.has_next()
    x, y, p = (np.zeros((2, 16), np.int32) for _ in range(3))
    dl.load_batch(x, y, p)
    assert dl.seq_len == 16 and (x[:, 1:] == y[:, :-1]).all() and (p[0] == np.arange(16)).all()
    first = x.copy()
    dl2 = DataLoader([shard], chunk_size=2 * 16, seed=5)
    dl2.load_batch(x, y)
    assert (x == first).all()                      # same seed, same first batch
    with pytest.raises(ValueError, match="chunks of 32"):
        dl.load_batch(np.zeros((4, 16), np.int32), np.zeros((4, 16), np.int32))
    assert not dl.has_kd()
    with pytest.raises(RuntimeError):
        dl.enable_kd(4)


def test_architecture_presets(tmp_path):
    from surogate_b200.config.sft_config import SFTConfig
    from surogate_b200.dsl.compiler import compile_model, model_from_hf_config
    from surogate_b200.models.presets import PRESETS, list_presets, normalise, preset_config
    from surogate_b200.train.sft import resolve_model_config

    assert normalise("Qwen/Qwen3-8B") == "qwen3-8b" and normalise("preset:meta-llama/Llama-3.1-8B-Instruct") == "llama-3.1-8b" and "qwen3-30b-a3b" in list_presets()
    c = PretrainedConfig.from_name("Qwen/Qwen3-8B")
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.intermediate_size, c.head_size) == (4096, 36, 32, 8, 12288, 128)
    assert not c.tie_word_embeddings and PretrainedConfig.from_name("qwen3-0.6b").tie_word_embeddings
    with pytest.raises(KeyError, match="known:"):
        preset_config("gpt-5")
    # every preset builds a model of the named size (parameter counts within 3% of the names)
    expect = {"qwen3-0.6b": 0.6, "qwen3-8b": 8.2, "qwen3-32b": 32.8, "qwen3-30b-a3b": 30.5, "qwen2.5-7b": 7.6, "llama-3.1-8b": 8.0, "llama-3.2-1b": 1.24, "mistral-7b-v0.3": 7.25}
    for name in PRESETS:
        cm = compile_model(model_from_hf_config(preset_config(name)))
        billions = cm.num_parameters() / 1e9
        if name in expect:
            assert abs(billions - expect[name]) / expect[name] < 0.03, (name, billions)
    cfg = SFTConfig.from_dict(dict(model="preset:qwen3-0.6b", synthetic_data=True, from_scratch=True, lora=False, tokenizer_path=str(tmp_path)))
    assert resolve_model_config(cfg)["hidden_size"] == 1024
    from surogate_b200.train.tokenize import tokenizer_dir

    assert tokenizer_dir(cfg) == str(tmp_path) and tokenizer_dir(SFTConfig.from_dict(dict(model="preset:qwen3-0.6b", synthetic_data=True))) is None

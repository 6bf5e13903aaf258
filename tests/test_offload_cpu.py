"""Host-resident state (offload_master / offload_optimizer / cpu_training) follows the same trajectory as the plain path."""
import numpy as np
import pytest
import torch

from surogate_b200.runtime.trainer import Trainer, TrainerConfig

MODEL = dict(architecture="Qwen3ForCausalLM", vocab_size=256, d_model=64, n_layers=2, num_query_heads=4, num_kv_heads=2, head_size=16, d_ff=128,
             tie_word_embeddings=True)


def _run(steps=3, **kw):
    cfg = TrainerConfig(model=MODEL, batch_size=2, seq_len=32, recipe="bf16", learning_rate=1e-2, weight_decay=0.1, zero_level=0, **kw)
    tr = Trainer(cfg, device=torch.device("cpu"))
    tr.init_weights(seed=3)
    rng = np.random.default_rng(0)
    out = []
    for _ in range(steps):
        tok = rng.integers(0, 256, (2, 33)).astype(np.int32)
        out.append(tr.step(tok[:, :-1], tok[:, 1:]))
    return tr, out


@pytest.mark.parametrize("opt", ["adamw", "adamw_8bit"])
def test_streamed_optimizer_matches_plain(opt):
    _, base = _run(optimizer=opt)
    tr, off = _run(optimizer=opt, offload_master=True, offload_optimizer=True)
    for a, b in zip(base, off):
        assert abs(a["loss"] - b["loss"]) < 1e-6 and abs(a["norm"] - b["norm"]) < 1e-6
    assert tr.streamed is not None


def test_cpu_training_matches_adamw():
    _, base = _run(optimizer="adamw")
    tr, cpu = _run(optimizer="adamw", cpu_training=True)
    for a, b in zip(base, cpu):
        assert abs(a["loss"] - b["loss"]) < 2e-5, (a, b)
    assert type(tr.optimizer).__name__ == "CpuAdamW"
    assert all(b.master.dtype == torch.float32 for b in tr.store.buckets.values())


def test_lora_with_host_resident_base():
    lora = dict(rank=4, alpha=8, dropout=0.0, dtype="fp32", targets=["q_proj", "v_proj", "down_proj"], rslora=False, train_router=False)
    _, base = _run(optimizer="adamw", lora=lora)
    _, off = _run(optimizer="adamw", lora=lora, offload_master=True, offload_optimizer=True)
    for a, b in zip(base, off):
        assert abs(a["loss"] - b["loss"]) < 1e-6


def test_resident_layers_keep_frozen_weights_on_the_device_side():
    """With offloaded masters the first N layers' frozen weights can stay resident: same trajectory, and the flag only applies to
    frozen layer buckets."""
    lora = dict(rank=4, alpha=8, dropout=0.0, dtype="fp32", targets=["q_proj", "v_proj", "down_proj"], rslora=False, train_router=False)
    tr_a, a = _run(optimizer="adamw", lora=lora, offload_master=True, offload_optimizer=True)
    tr_b, b = _run(optimizer="adamw", lora=lora, offload_master=True, offload_optimizer=True, resident_layers=1)
    assert a == b
    st = tr_b.store
    assert st._resident(st.buckets["layer0"]) and not st._resident(st.buckets["layer1"]) and not st._resident(st.buckets["embedding"])


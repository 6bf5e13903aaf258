"""LoRA on CPU: adapter gradients against autograd, frozen base, PEFT export round trip, merge."""
import json
import os

import numpy as np
import torch

from surogate_b200.runtime.trainer import Trainer, TrainerConfig

MODEL = dict(architecture="Qwen3ForCausalLM", vocab_size=256, d_model=64, n_layers=2, num_query_heads=4, num_kv_heads=2, head_size=16, d_ff=128,
             tie_word_embeddings=False)


def _trainer(**lora):
    cfg = TrainerConfig(model=MODEL, batch_size=2, seq_len=32, optimizer="adamw", learning_rate=1e-2,
                        lora=dict(rank=4, alpha=8, targets=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"], **lora))
    tr = Trainer(cfg)
    tr.init_weights(0)
    return tr


def _batch():
    rng = np.random.default_rng(0)
    tok = rng.integers(0, 256, (2, 33)).astype(np.int32)
    return tok[:, :-1], tok[:, 1:]


def test_lora_trains_only_adapters_and_loss_drops(tmp_path):
    tr = _trainer()
    base_before = {n: t.clone() for n, t in tr.store.named_full_tensors()}
    x, y = _batch()
    losses = [tr.step(x, y)["loss"] for _ in range(10)]
    assert losses[-1] < losses[0] - 0.05, losses
    for n, t in tr.store.named_full_tensors():
        assert torch.equal(t, base_before[n]), f"base parameter {n} changed under LoRA"
    # PEFT export
    out = tmp_path / "adapter"
    tr.export_adapter(str(out))
    cfg = json.load(open(out / "adapter_config.json"))
    assert cfg["r"] == 4 and cfg["peft_type"] == "LORA" and "q_proj" in cfg["target_modules"]
    from safetensors import safe_open

    with safe_open(str(out / "adapter_model.safetensors"), framework="pt") as f:
        keys = set(f.keys())
        a = f.get_tensor("base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight")
        b = f.get_tensor("base_model.model.model.layers.1.mlp.down_proj.lora_B.weight")
    assert a.shape == (4, 64) and b.shape == (64, 4) and len(keys) == 2 * 7 * 2
    # round trip into a fresh trainer reproduces the loss
    tr2 = _trainer()
    tr2.lora.load_peft(str(out))
    l1 = tr.validate(x, y)["loss"]
    l2 = tr2.validate(x, y)["loss"]
    assert abs(l1 - l2) < 1e-5


def test_lora_gradients_match_autograd():
    tr = _trainer()
    # give B non-zero values so that gradients flow to A as well
    g = torch.Generator().manual_seed(3)
    tr.lora.master.add_(0.05 * torch.randn(tr.lora.numel, generator=g))
    tr.lora.sync_work()
    x, y = _batch()
    tr.forward_backward(x, y)
    grad = tr.lora.grad.clone()
    # autograd oracle: merge the adapters into dense weights as differentiable functions of the flat buffer
    from torch_reference import model_loss

    flat = tr.lora.master.clone().requires_grad_(True)
    p = {n: t.clone() for n, t in tr.store.named_full_tensors()}
    for grp in tr.lora.groups.values():
        name = f"blocks.{grp.layer}.{grp.param}"
        w = p[name]
        pieces = []
        covered = 0
        for t in grp.targets:
            A = flat[t.a_off:t.a_off + 4 * grp.in_features].view(4, grp.in_features)
            B = flat[t.b_off:t.b_off + t.rows * 4].view(t.rows, 4)
            pieces.append(w[t.row_off:t.row_off + t.rows] + tr.lora.scaling * (B @ A))
            covered += t.rows
        assert covered == w.shape[0]
        p[name] = torch.cat(pieces, 0)
    T = 32
    pos = torch.arange(T)[None].expand(2, T)
    cfg = dict(n_layers=2, Hq=4, Hkv=2, D=16, eps=1e-6, theta=1e6)
    loss, _ = model_loss(p, torch.from_numpy(x).long(), pos, torch.from_numpy(y), cfg)
    (loss / (2 * T)).backward()
    assert torch.allclose(grad, flat.grad, rtol=1e-4, atol=1e-6), (grad - flat.grad).abs().max()


def test_merge_adapter_equals_adapted_forward():
    tr = _trainer()
    tr.lora.master.add_(0.05 * torch.randn(tr.lora.numel, generator=torch.Generator().manual_seed(1)))
    tr.lora.sync_work()
    x, y = _batch()
    adapted = tr.validate(x, y)["loss"]
    tr.lora.merge_into(tr.store)
    tr.executor.lora = None
    merged = tr.validate(x, y)["loss"]
    assert abs(adapted - merged) < 1e-5


def test_lora_checkpoint_holds_only_the_adapter_and_resumes_with_dropout(tmp_path):
    """A LoRA checkpoint leaves the frozen base out; a fresh trainer whose base was re-created from the same seed continues the
    run exactly, including the dropout masks (the generator state is part of the checkpoint)."""
    from safetensors import safe_open

    x, y = _batch()
    tr = _trainer(dropout=0.2)
    for _ in range(3):
        tr.step(x, y)
    d = tr.save_checkpoint(str(tmp_path), step=3)
    with safe_open(os.path.join(d, "weights.shard_000_of_001.safetensors"), framework="pt") as f:
        assert not [k for k in f.keys() if k != "__empty__"]
    assert os.path.getsize(os.path.join(d, "weights.shard_000_of_001.safetensors")) < 4096
    cont = [tr.step(x, y)["loss"] for _ in range(3)]
    torch.manual_seed(12345)  # a resumed process starts from some other generator state
    tr2 = _trainer(dropout=0.2)
    tr2.load_checkpoint(str(tmp_path))
    assert [tr2.step(x, y)["loss"] for _ in range(3)] == cont

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


MOE_MODEL = dict(architecture="Qwen3MoeForCausalLM", vocab_size=256, d_model=64, n_layers=2, num_query_heads=4, num_kv_heads=2, head_size=16,
                 moe_d_ff=32, num_experts=4, num_experts_per_tok=2, aux_loss_coef=0.0, tie_word_embeddings=False)


def _moe_trainer(lora=True, seed=0):
    kw = dict(lora=dict(rank=4, alpha=8, dropout=0.0, dtype="fp32", targets=["q_proj", "v_proj", "gate_proj", "up_proj", "down_proj"])) if lora else {}
    cfg = TrainerConfig(model=MOE_MODEL, batch_size=2, seq_len=32, optimizer="adamw", learning_rate=1e-2, zero_level=0, **kw)
    tr = Trainer(cfg)
    tr.init_weights(seed)
    return tr


def test_expert_lora_gradients_follow_the_chain_rule_through_merged_weights(tmp_path):
    """Per-expert adapters on the grouped expert projections: the adapted forward equals the forward with merged weights, the
    adapter gradients equal s * B^T dW and s * dW A^T of the merged model's full weight gradient (exact chain rule), training lowers
    the loss with the base frozen, and the PEFT export / import round-trips the per-expert keys."""
    tr = _moe_trainer()
    experts = [g for g in tr.lora.groups.values() if g.experts]
    assert {g.param for g in experts} == {"experts_gate_up", "experts_down"} and all(g.experts == 4 for g in experts)
    tr.lora.master.add_(0.05 * torch.randn(tr.lora.numel, generator=torch.Generator().manual_seed(3)))
    tr.lora.sync_work()
    x, y = _batch()
    adapted = tr.validate(x, y)["loss"]
    tr.forward_backward(x, y)
    grad = tr.lora.grad.clone()
    # the same model without adapters, holding the merged weights, trained in full
    full = _moe_trainer(lora=False)
    merged = _moe_trainer()
    merged.lora.master.copy_(tr.lora.master)
    merged.lora.merge_into(merged.store)
    for name, t in merged.store.named_full_tensors():
        full.store.load_tensor(name, t.cpu())
    full.store.sync_work_from_master()
    assert abs(full.validate(x, y)["loss"] - adapted) < 1e-5
    full.forward_backward(x, y)
    dW = full.get_gradients()
    s = tr.lora.scaling
    for g in experts:
        w_grad = dW[f"blocks.{g.layer}.{g.param}"].float()
        for t in g.targets:
            A, B = tr.lora._EA(tr.lora.master, g, t).float(), tr.lora._EB(tr.lora.master, g, t).float()
            sl = w_grad[:, t.row_off:t.row_off + t.rows]                     # [E, rows, K]
            want_a = s * torch.bmm(B.transpose(1, 2), sl)                     # [E, r, K]
            want_b = s * torch.bmm(sl, A.transpose(1, 2))                     # [E, rows, r]
            got_a, got_b = tr.lora._EA(grad, g, t), tr.lora._EB(grad, g, t)
            assert torch.allclose(got_a, want_a, rtol=2e-4, atol=1e-6), (g.param, t.name, (got_a - want_a).abs().max())
            assert torch.allclose(got_b, want_b, rtol=2e-4, atol=1e-6), (g.param, t.name, (got_b - want_b).abs().max())
    # training: adapters move, the base does not
    base_before = {n: t.clone() for n, t in tr.store.named_full_tensors()}
    losses = [tr.step(x, y)["loss"] for _ in range(8)]
    assert losses[-1] < losses[0] - 0.02, losses
    for n, t in tr.store.named_full_tensors():
        assert torch.equal(t, base_before[n]), n
    # PEFT round trip with per-expert keys
    out = tmp_path / "adapter"
    tr.export_adapter(str(out))
    from safetensors import safe_open

    with safe_open(str(out / "adapter_model.safetensors"), framework="pt") as f:
        keys = set(f.keys())
        a = f.get_tensor("base_model.model.model.layers.1.mlp.experts.3.up_proj.lora_A.weight")
        b = f.get_tensor("base_model.model.model.layers.0.mlp.experts.0.down_proj.lora_B.weight")
    assert a.shape == (4, 64) and b.shape == (64, 4)
    assert len([k for k in keys if ".experts." in k]) == 2 * 4 * 3 * 2   # layers x experts x (gate, up, down) x (A, B)
    tr2 = _moe_trainer()
    tr2.lora.load_peft(str(out))
    assert abs(tr.validate(x, y)["loss"] - tr2.validate(x, y)["loss"]) < 1e-5

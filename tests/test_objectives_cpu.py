"""Sequence-level objectives through the fused LM-head loss hooks: per-token weights (DPO / GRPO) and top-K distillation."""
import numpy as np
import torch

from surogate_b200.dpo.loss import dpo_loss_and_weights
from surogate_b200.runtime.trainer import Trainer, TrainerConfig

MODEL = dict(architecture="Qwen3ForCausalLM", vocab_size=128, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64,
             tie_word_embeddings=False)


def _trainer(**kw):
    cfg = TrainerConfig(model=MODEL, batch_size=4, seq_len=12, recipe="bf16", optimizer="adamw", learning_rate=1e-2, zero_level=0, max_grad_norm=0.0, **kw)
    tr = Trainer(cfg, device=torch.device("cpu"))
    tr.init_weights(seed=1)
    return tr


def _data(seed=0, rows=4, T=12, V=128):
    rng = np.random.default_rng(seed)
    tok = rng.integers(0, V, (rows, T + 1)).astype(np.int32)
    y = tok[:, 1:].copy()
    y[:, :4] = -100
    return tok[:, :-1], y


def _torch_params(tr):
    return {n: t.detach().clone().double().requires_grad_(True) for n, t in tr.store.named_full_tensors()}


def _logits(p, x):
    from torch_reference import model_logits

    return model_logits(p, torch.from_numpy(x).long(), dict(V=128, n_layers=1, Hq=2, Hkv=1, D=16, eps=1e-6, theta=1e6))


def test_dpo_gradient_matches_autograd():
    tr = _trainer()
    x, y = _data()
    pol = tr.token_logprobs(x, y).sum(1)
    ref = pol.detach() + torch.tensor([0.3, -0.2, 0.1, 0.4])
    loss, w_c, w_r, _ = dpo_loss_and_weights(pol[0::2], pol[1::2], ref[0::2], ref[1::2], beta=0.5)
    row_w = torch.stack([w_c, w_r], 1).reshape(-1)[:, None].expand(-1, 12).contiguous()
    tr.forward_backward(x, y, row_weights=row_w, loss_scale_override=1.0)
    # autograd reference of the same objective
    p = _torch_params(tr)
    lg = _logits(p, x)
    lp = torch.log_softmax(lg, -1)
    yt = torch.from_numpy(y).long()
    tokl = lp.gather(2, yt.clamp_min(0)[..., None]).squeeze(2) * (yt != -100)
    seq = tokl.sum(1)
    assert torch.allclose(seq.float(), pol, atol=1e-4)
    h = 0.5 * ((seq[0::2] - seq[1::2]) - (ref[0::2] - ref[1::2]).double())
    ref_loss = -torch.nn.functional.logsigmoid(h).mean()
    ref_loss.backward()
    assert abs(float(ref_loss) - float(loss)) < 1e-5
    for name, t in p.items():
        g = tr.store.grad_of(name)
        assert torch.allclose(g.double(), t.grad, atol=2e-5, rtol=1e-4), name


def test_topk_distillation_gradient_matches_autograd():
    tr = _trainer()
    x, y = _data(3)
    K = 5
    gen = torch.Generator().manual_seed(0)
    teacher = torch.log_softmax(torch.randn(4, 12, 128, generator=gen) * 2, -1)
    kl, ki = teacher.topk(K, dim=-1)
    kd = {"idx": ki.to(torch.int32), "logp": kl, "weight": 0.7, "ce_weight": 0.3}
    n_valid = float((y != -100).sum())
    r = tr.forward_backward(x, y, kd=kd)
    p = _torch_params(tr)
    lp = torch.log_softmax(_logits(p, x), -1)
    yt = torch.from_numpy(y).long()
    valid = (yt != -100)
    ce = -(lp.gather(2, yt.clamp_min(0)[..., None]).squeeze(2) * valid).sum()
    kdl = ((kl.double().exp() * (kl.double() - lp.gather(2, ki))).sum(-1) * valid).sum()
    total = (0.3 * ce + 0.7 * kdl) / n_valid
    total.backward()
    assert abs(float(r["loss_sum"]) / n_valid - float(total)) < 1e-5
    for name, t in p.items():
        g = tr.store.grad_of(name)
        assert torch.allclose(g.double(), t.grad, atol=2e-5, rtol=1e-4), name


def test_dpo_step_improves_margin_with_lora_reference():
    lora = dict(rank=4, alpha=8, dropout=0.0, dtype="fp32", targets=["q_proj", "v_proj", "o_proj", "up_proj", "down_proj"], rslora=False, train_router=False)
    tr = _trainer(lora=lora)
    from surogate_b200.dpo.trainer import DPOTrainer

    dpo = DPOTrainer(tr, beta=0.5)
    x, y = _data(5)
    hist = [dpo.step(x, y, lr=5e-2) for _ in range(12)]
    assert abs(hist[0]["rewards/margin"]) < 1e-6  # adapters start as identity: policy == reference
    assert hist[-1]["rewards/margin"] > 0.05 and hist[-1]["loss"] < hist[0]["loss"]


def test_phase_timing_reports_forward_head_backward_and_optimizer():
    import numpy as np
    import torch

    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    model = dict(architecture="Qwen3ForCausalLM", vocab_size=200, d_model=32, n_layers=2, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64, tie_word_embeddings=True)
    tr = Trainer(TrainerConfig(model=model, batch_size=1, grad_accum=2, seq_len=16, zero_level=0, time_breakdown=True), device=torch.device("cpu"))
    tr.init_weights(seed=0)
    tok = np.random.default_rng(0).integers(0, 200, (2, 17)).astype(np.int32)
    tr.step(tok[:, :-1], tok[:, 1:])
    t = tr.last_time_breakdown
    assert set(t) == {"forward_ms", "lm_head_ms", "backward_ms", "optimizer_ms"} and all(v > 0 for v in t.values())
    tr.step(tok[:, :-1], tok[:, 1:])
    assert tr.last_time_breakdown["forward_ms"] < 10 * t["forward_ms"] + 50  # marks are reset per step, not accumulated over the run


def test_gradient_masks_train_only_what_they_allow():
    """Partial-update runs of a full model: with an allow-list only the named parameters change; with the MLP-growth mask only
    the new half of each MLP matrix changes (and is not decayed), everything else stays bit-identical."""
    import torch

    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    model = dict(architecture="Qwen3ForCausalLM", vocab_size=128, d_model=32, n_layers=2, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64)
    tok = torch.randint(0, 128, (2, 17), generator=torch.Generator().manual_seed(0))

    def run(**kw):
        tr = Trainer(TrainerConfig(model=model, batch_size=2, seq_len=16, zero_level=0, optimizer="adamw", weight_decay=0.1, learning_rate=1e-2, **kw),
                     device=torch.device("cpu"))
        tr.init_weights(0)
        before = {n: tr.store.get(n).clone() for n in tr.store.where}
        for _ in range(2):
            tr.step(tok[:, :-1].numpy(), tok[:, 1:].numpy())
        return before, {n: tr.store.get(n).clone() for n in tr.store.where}

    before, after = run(trainable_param_substrings=["qkv_weight", "final_norm"])
    for n in before:
        changed = not torch.equal(before[n], after[n])
        assert changed == ("qkv_weight" in n or "final_norm" in n), n

    before, after = run(gradient_mask_mode="mlp_growth_new_half")
    for n in before:
        d = (after[n] - before[n]).abs()
        if "mlp_up_weight" in n:
            q = d.shape[0] // 4
            assert d[:q].max() == 0 and d[2 * q:3 * q].max() == 0 and d[q:2 * q].max() > 0 and d[3 * q:].max() > 0, n
        elif "mlp_down_weight" in n:
            h = d.shape[1] // 2
            assert d[:, :h].max() == 0 and d[:, h:].max() > 0, n
        else:
            assert d.max() == 0, n

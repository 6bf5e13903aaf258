"""GRPO pieces on CPU: token-weight gradient vs autograd, packer alignment, transport, orchestrator with a fake engine."""
import numpy as np
import torch

from surogate_b200.grpo.loss import group_advantages, grpo_loss_reference, grpo_token_weights
from surogate_b200.grpo.packer import Rollout, pack_rollouts


def test_token_weights_equal_autograd_gradient():
    torch.manual_seed(0)
    logp = (torch.randn(3, 10) * 0.5 - 2).requires_grad_(True)
    old = logp.detach() + torch.randn(3, 10) * 0.3
    ref = logp.detach() + torch.randn(3, 10) * 0.2
    adv = torch.randn(3, 1).expand(3, 10).contiguous()
    mask = torch.rand(3, 10) > 0.3
    seq = torch.arange(3)[:, None].expand(3, 10).contiguous()
    for norm in ("token", "sequence"):
        loss, _ = grpo_loss_reference(logp, old, adv, mask, ref, 0.2, 0.28, 0.05, 10.0, norm, seq)
        (g,) = torch.autograd.grad(loss, logp)
        l2, w, m = grpo_token_weights(logp.detach(), old, adv, mask, ref, 0.2, 0.28, 0.05, 10.0, norm, seq)
        assert torch.allclose(loss.detach(), l2, atol=1e-6)
        assert torch.allclose(w, -g, atol=1e-6), norm  # the kernel scales dCE = -dlogp by w
        assert 0 <= float(m["clip_frac"]) <= 1


def test_group_advantages():
    a = group_advantages(torch.tensor([1.0, 0.0, 0.0, 1.0, 2.0, 2.0, 2.0, 2.0]), 4)
    assert torch.allclose(a[:4], torch.tensor([1.0, -1.0, -1.0, 1.0]), atol=1e-4) and torch.all(a[4:] == 0)


def test_packer_aligns_targets_logprobs_and_resets_positions():
    r1 = Rollout([1, 2, 3], [4, 5], [-0.1, -0.2], advantage=0.5)
    r2 = Rollout([7], [8, 9, 10], [-1.0, -1.1, -1.2], advantage=-1.0)
    (b,) = pack_rollouts([r1, r2], seq_len=12, rows=1)
    x, y, p = b.inputs[0], b.targets[0], b.position_ids[0]
    assert list(x[:9]) == [1, 2, 3, 4, 5, 7, 8, 9, 10]
    assert list(p[:9]) == [0, 1, 2, 3, 4, 0, 1, 2, 3]
    # position 2 (token 3) predicts 4, position 3 predicts 5; position 5 (token 7) predicts 8 ...
    assert list(y[:9]) == [-100, -100, 4, 5, -100, 8, 9, 10, -100]
    assert np.allclose(b.old_logprobs[0][[2, 3, 5, 6, 7]], [-0.1, -0.2, -1.0, -1.1, -1.2])
    assert np.allclose(b.advantages[0][[2, 3]], 0.5) and np.allclose(b.advantages[0][[5, 6, 7]], -1.0)
    assert list(b.seq_ids[0][:9]) == [0] * 5 + [1] * 4 and (b.seq_ids[0][9:] == -1).all()
    assert (y[9:] == -100).all()


class _FakeTok:
    pad_token_id = 0

    def apply_chat_template_and_encode(self, msgs, add_generation_prompt=True):
        return [1] + [ord(c) % 50 + 2 for c in msgs[-1]["content"]][:6]


class _FakeEngine:
    def __init__(self):
        self.calls = 0

    def generate(self, prompt_ids, n, sampling):
        self.calls += 1
        out = []
        for k in range(n):
            ids = [10 + k] * (2 + k % 3)
            out.append((ids, [-0.5] * len(ids), "42" if k % 2 == 0 else "7"))
        return out


def test_orchestrator_end_to_end_with_fake_engine(tmp_path):
    from surogate_b200.grpo.config import OrchestratorConfig
    from surogate_b200.grpo.orchestrator import Orchestrator
    from surogate_b200.grpo.transport import FilesystemTransport

    cfg = OrchestratorConfig(group_size=4, prompts_per_step=2, sequence_len=48, rows_per_step=2, max_steps=3, max_async_level=1,
                             transport_dir=str(tmp_path))
    tr = FilesystemTransport(str(tmp_path))
    version = {"v": 0}
    orch = Orchestrator(cfg, _FakeTok(), _FakeEngine(), tr, lambda: version["v"])
    orch.load_prompts([{"prompt": "what is 6*7", "answer": "42"}, {"prompt": "what is 40+2", "answer": "42"}])
    st0, st1 = orch.run_step(0), orch.run_step(1)
    assert st0.groups_kept == 2 and abs(st0.reward_mean - 0.5) < 1e-6
    arrays, meta = tr.receive(0, timeout_s=1)
    assert arrays["inputs"].shape == (2, 48) and meta["n_samples"] == 8
    valid = arrays["targets"] != -100
    assert valid.sum() > 0 and np.all(arrays["old_logprobs"][valid] == -0.5)
    assert set(np.unique(np.round(arrays["advantages"][valid], 3))) == {-1.0, 1.0}
    # depth control: step 2 needs policy version >= 1
    orch.depth.timeout = 0.2
    try:
        orch.run_step(2)
        raise AssertionError("should have waited for the trainer")
    except TimeoutError:
        pass
    version["v"] = 1
    assert orch.run_step(2).policy_version == 1
    tr.ack(1)
    tr.cleanup(tr.acked())
    assert not tr.ready(0) and tr.ready(1)


def test_grpo_trainer_step_raises_rewarded_tokens(tmp_path):
    from surogate_b200.grpo.trainer import GRPOTrainer
    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    model = dict(architecture="Qwen3ForCausalLM", vocab_size=64, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64,
                 tie_word_embeddings=True)
    t = Trainer(TrainerConfig(model=model, batch_size=2, seq_len=16, recipe="bf16", optimizer="adamw", learning_rate=2e-2, zero_level=0),
                device=torch.device("cpu"))
    t.init_weights(seed=0)
    g = GRPOTrainer(t)
    good = Rollout([1, 2, 3], [20, 21, 22], [0.0, 0.0, 0.0], advantage=1.0)
    bad = Rollout([1, 2, 3], [30, 31, 32], [0.0, 0.0, 0.0], advantage=-1.0)

    def batch():
        (b,) = pack_rollouts([good, bad], 16, 2)
        arr = b.arrays()
        lp = t.token_logprobs(arr["inputs"], arr["targets"], arr["position_ids"]).cpu().numpy()
        arr["old_logprobs"] = np.where(arr["targets"] != -100, lp, 0).astype(np.float32)  # on-policy rollouts
        return arr, lp

    arr, lp0 = batch()
    for _ in range(5):
        out = g.step(arr)
        arr, lp = batch()
    m = arr["targets"] != -100
    adv = arr["advantages"]
    assert (lp[m & (adv > 0)].sum() > lp0[m & (adv > 0)].sum()) and (lp[m & (adv < 0)].sum() < lp0[m & (adv < 0)].sum())
    assert np.isfinite(out["loss"]) and out["ratio_mean"] > 0

"""GRPO pieces on CPU: token-weight gradient vs autograd, packer alignment, transport, orchestrator with a fake engine."""
import numpy as np
import pytest
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


def test_environments_generate_verify_and_evaluate(tmp_path):
    """Three built-in environments: gold answers are recomputed from the data, an oracle policy scores 1, a wrong one 0, the
    tool loop feeds lookups back, and a scaffolded environment loads and evaluates."""
    import json as _json
    import os
    import re as _re

    from surogate_b200.cli.vf import init_environment
    from surogate_b200.grpo.environments import as_reward_fn, evaluate, load_environment
    from surogate_b200.grpo.environments import markdown_table_qa as mt

    env = load_environment("markdown-table-qa", num_train=40, num_eval=12, seed=1)
    by_q = {e["prompt"][0]["content"]: e for e in env.dataset + env.eval_dataset}

    def oracle(msgs):
        e = by_q[msgs[-1]["content"]]
        return f"<think>work</think>\n{e['answer']}"

    assert msgs_have_system(env, oracle)
    r = evaluate(env, oracle, 12, 1)
    assert r["mean_reward"] > 0.99 and r["n"] == 12
    assert evaluate(env, lambda m: "<think>hm</think>\nbanana -1", 12)["mean_reward"] < 0.05
    df = mt.parse_markdown_table("| Name | Region | Revenue | Units |\n|---|---|---|---|\n| A | North | 10 | 1 |\n| B | South | 30 | 2 |")
    assert list(df.columns) == ["Name", "Region", "Revenue", "Units"] and len(df) == 2
    assert mt.compute_gold("| Name | Region | Revenue | Units |\n|---|---|---|---|\n| A | North | 10 | 1 |\n| B | South | 30 | 2 |", "percentage", "Revenue", "South")["value"] == 75.0
    assert mt.correctness_reward("<think>x</think> 75.2", 75.0, {"qtype": "percentage"}) == 1.0
    assert 0 < mt.correctness_reward("the answer is 60", 75.0, {"qtype": "sum"}) < 1
    scores = as_reward_fn(env)(env.dataset[0], [oracle(env.initial_messages(env.dataset[0])), "no idea"])
    assert scores[0] > 0.99 and scores[1] < 0.5

    tools = load_environment("multihop-tools", num_train=4, num_eval=4, hops=3, seed=2)

    def tool_user(msgs):  # follows the chain with lookups, then answers
        ex = next(e for e in tools.eval_dataset + tools.dataset if e["prompt"][0]["content"] == msgs[1]["content"])
        q = ex["prompt"][0]["content"]
        field = _re.match(r"What is the (\w+) of", q).group(1)
        rels = list(reversed(_re.findall(r"the (\w+) of", q)[1:]))
        start = _re.search(r"of ([A-Z]\w* \w+)\?$", q).group(1)
        results = [m["content"] for m in msgs if m["role"] == "tool"]
        ent = start if not results else results[-1]
        k = len(results)
        if k < len(rels):
            return '<tool>{"name": "lookup", "args": {"entity": "%s", "field": "%s"}}</tool>' % (ent, rels[k])
        if k == len(rels):
            return '<tool>{"name": "lookup", "args": {"entity": "%s", "field": "%s"}}</tool>' % (ent, field)
        return f"<answer>{results[-1]}</answer>"

    r2 = evaluate(tools, tool_user, 4)
    assert r2["mean_reward"] == 1.0 and all(s["turns"] == 4 for s in r2["samples"])
    assert evaluate(tools, lambda m: "<answer>nowhere</answer>", 4)["mean_reward"] == 0.0

    data = tmp_path / "rows.jsonl"
    data.write_text("\n".join(_json.dumps({"question": f"capital of country {i}?", "answer": f"city{i}"}) for i in range(5)))
    ruler = load_environment("ruler-task", dataset_path=str(data), user_template="Q: {question}", system_prompt="Be brief.")
    assert ruler.dataset[2]["prompt"][0]["content"] == "Q: capital of country 2?"
    assert ruler.score_group(ruler.dataset[2], ["it is city2", "unknown"]) == [1.0, 0.0]

    root = init_environment("my-task", str(tmp_path / "envs"))
    assert sorted(os.listdir(root)) == ["README.md", "my_task.py", "pyproject.toml"]
    mine = load_environment("my-task", path=str(tmp_path / "envs"))
    assert evaluate(mine, lambda m: "4", 1)["mean_reward"] == 1.0


def msgs_have_system(env, policy):
    msgs = env.initial_messages(env.dataset[0])
    return msgs[0]["role"] == "system" and msgs[-1]["role"] == "user" and isinstance(policy(msgs), str)


def test_orchestrator_runs_multi_turn_tool_episodes(tmp_path):
    """A multi-turn environment drives episodes: assistant turns are sampled one by one, tool replies are inserted as context
    tokens that carry no loss, and the episode's reward becomes the advantage of every assistant token."""
    import json as _json

    from surogate_b200.grpo.config import OrchestratorConfig
    from surogate_b200.grpo.orchestrator import Orchestrator
    from surogate_b200.grpo.transport import FilesystemTransport

    class Tok:  # one token per character, messages joined by a separator token; re-encoding is prefix-stable
        pad_token_id = 0

        def apply_chat_template_and_encode(self, msgs, add_generation_prompt=True):
            ids = []
            for m in msgs:
                ids += [1] + [ord(c) + 10 for c in m["content"]] + ([2] if m["role"] != "assistant" else [])
            return ids + ([3] if add_generation_prompt else [])

    tok = Tok()

    class Engine:  # even episodes follow the lookups and answer correctly, odd ones answer wrongly at once
        def __init__(self):
            self.k = 0
            self.turn = {}

        def generate(self, prompt_ids, n, sampling):
            text = "".join(chr(t - 10) for t in prompt_ids if t >= 10)
            episode = self.k
            if "RESULT" not in text and not self.turn.get(episode):
                self.turn[episode] = 1
                reply = '<tool>{"name": "lookup", "args": {"entity": "E", "field": "city"}}</tool>' if episode % 2 == 0 else "<answer>nowhere</answer>"
            else:
                reply = "<answer>Oslo</answer>"
            if "<answer>" in reply:
                self.k += 1
            ids = [ord(c) + 10 for c in reply] + [4]  # 4 = end of turn, part of the sampled tokens
            return [(ids, [-0.25] * len(ids), reply)]

    from surogate_b200.grpo.environments.base import MultiTurnEnv, Rubric

    class Env(MultiTurnEnv):
        env_id = "toy-tools"

        def is_completed(self, messages, state):
            return "<answer>" in messages[-1]["content"]

        def env_response(self, messages, state):
            return [{"role": "tool", "content": "RESULT Oslo"}]

    def correct(completion, answer, **_):
        return 1.0 if f"<answer>{answer}</answer>" in completion else 0.0

    cfg = OrchestratorConfig(group_size=4, prompts_per_step=1, sequence_len=400, rows_per_step=2, max_steps=1, transport_dir=str(tmp_path), max_tokens=64)
    orch = Orchestrator(cfg, tok, Engine(), FilesystemTransport(str(tmp_path)), lambda: 0)
    orch.env = Env([{"prompt": [{"role": "user", "content": "city of E?"}], "answer": "Oslo"}], Rubric([correct]), max_turns=4)
    orch.load_prompts()

    class PrefixTok(Tok):  # the sampled end-of-turn token 4 must reappear when the conversation is re-encoded
        def apply_chat_template_and_encode(self, msgs, add_generation_prompt=True):
            ids = []
            for m in msgs:
                ids += ([3] if m["role"] == "assistant" else [1]) + [ord(c) + 10 for c in m["content"]] + ([4] if m["role"] == "assistant" else [2])
            return ids + ([3] if add_generation_prompt else [])  # the generation prompt is the assistant header

    orch.tok = PrefixTok()
    rollouts, stats = orch.collect(0, 0)
    assert stats["groups_kept"] == 1 and abs(stats["reward_mean"] - 0.5) < 1e-9 and len(rollouts) == 4
    good = [r for r in rollouts if r.reward == 1.0]
    bad = [r for r in rollouts if r.reward == 0.0]
    assert len(good) == 2 and len(bad) == 2 and good[0].advantage > 0 > bad[0].advantage
    g = good[0]
    assert 0 in g.completion_mask and g.completion_mask[0] == 1 and g.completion_mask[-1] == 1  # tool reply in the middle is context
    n_env = g.completion_mask.count(0)
    assert n_env == len("RESULT Oslo") + 3  # [1] + text + [2] + generation prompt [3]
    assert all(m == 1 for m in bad[0].completion_mask)
    st = orch.run_step(0)
    arrays, meta = orch.transport.receive(0, timeout_s=1)
    trained = arrays["targets"] != -100
    assert trained.sum() == sum(sum(r.completion_mask) for r in rollouts) and np.all(arrays["old_logprobs"][trained] == -0.25)


def test_ipo_objective_weights_match_autograd_and_mask_drifted_tokens():
    """``type: ipo``: the per-token weights equal minus the autograd gradient of the surrogate; a token whose probability moved past
    the mask thresholds keeps only the penalty term; the ratio that multiplies the gradient is capped."""
    from surogate_b200.grpo.loss import ipo_loss_reference, ipo_token_weights

    torch.manual_seed(0)
    R, T = 3, 12
    old = -torch.rand(R, T) * 2.0 - 0.05
    logp = (old + 0.3 * torch.randn(R, T)).clamp(max=-1e-3)
    logp[0, 0], old[0, 0] = -0.05, -2.5      # probability rose by ~0.87 > 0.2: masked (high)
    logp[0, 1], old[0, 1] = -3.0, -0.1       # fell by ~0.85: masked (low)
    logp[1, 2], old[1, 2] = -0.9, -3.2       # ratio ~10 > e^2 but probability difference 0.37 -> masked as well
    logp[2, 3], old[2, 3] = -4.0, -6.5       # ratio ~12, probability difference tiny: kept, ratio capped at e^2
    adv = torch.randn(R, T)
    teacher = old + 0.1 * torch.randn(R, T)
    mask = (torch.rand(R, T) > 0.2).float()
    mask[0, :2] = mask[1, 2] = mask[2, 3] = 1.0
    seq = torch.arange(R)[:, None].expand(R, T).contiguous()
    for kw in (dict(), dict(teacher_logp=teacher, teacher_tau=0.3, adv_tau=0.7, kl_tau=0.05), dict(normalization="sequence", seq_ids=seq)):
        lp = logp.clone().requires_grad_(True)
        ipo_loss_reference(lp, old, adv, mask, **kw).backward()
        loss, w, metrics = ipo_token_weights(logp, old, adv, mask, **kw)
        assert torch.allclose(w, -lp.grad, atol=1e-6), kw
        assert torch.isfinite(loss)
    loss, w, metrics = ipo_token_weights(logp, old, adv, mask, kl_tau=0.0)
    Z = mask.sum()
    for r, t in ((0, 0), (0, 1), (1, 2)):
        assert w[r, t] == 0.0                                     # masked tokens leave the policy term; no penalty with kl_tau 0
    assert torch.allclose(w[2, 3], adv[2, 3] * 7.389056 / Z, atol=1e-6)      # kept, capped ratio
    assert float(metrics["is_masked"]) >= 3.0 / float(Z) - 1e-6 and float(metrics["is_masked_high"]) > 0 and float(metrics["is_masked_low"]) > 0
    _, w2, _ = ipo_token_weights(logp, old, adv, mask, kl_tau=0.5)
    assert torch.allclose(w2[0, 0], -2 * 0.5 * (logp[0, 0] - old[0, 0]) / Z, atol=1e-6)   # the penalty still pulls a masked token back


def test_loss_section_selects_the_objective_and_trainer_keys_have_both_spellings():
    from surogate_b200.grpo.config import GRPOConfig, GRPOLossConfig

    assert GRPOLossConfig().type == "clip" and GRPOLossConfig(kl_tau=1e-2).type == "ipo" and GRPOLossConfig(type="ipo").ipo_mask_low == 0.2
    assert abs(GRPOLossConfig(type="ipo").ratio_clip - 7.389056) < 1e-9 and GRPOLossConfig(clip_eps_high=0.3).type == "clip"
    with pytest.raises(ValueError):
        GRPOLossConfig(type="dpo")
    model = dict(architecture="Qwen3ForCausalLM", vocab_size=64, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64, tie_word_embeddings=True)
    import json

    cfg = GRPOConfig.from_dict(dict(model=json.dumps(model), transport_type="zmq", weight_broadcast_type="nccl", max_async_level=1, turn_diagnostics=True,
                                    noise_scheduler=dict(enabled=True, sigma_start=0.05, sigma_end=0.0005, num_stages=4),
                                    loss=dict(ipo_mask_low=0.1, ipo_mask_high=0.3, kl_tau=0.01, adv_tau=1.0, teacher_tau=0.0, ratio_clip=5.0)))
    assert cfg.transport == "zmq" and cfg.weight_broadcast == "nccl" and cfg.loss.type == "ipo" and cfg.loss.ipo_mask_high == 0.3 and cfg.turn_diagnostics
    assert cfg.noise_scheduler["num_stages"] == 4


def test_grpo_trainer_step_with_the_ipo_objective_and_turn_diagnostics():
    from surogate_b200.grpo.config import GRPOLossConfig
    from surogate_b200.grpo.trainer import GRPOTrainer
    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    torch.manual_seed(0)
    tr = Trainer(TrainerConfig(model=dict(architecture="Qwen3ForCausalLM", vocab_size=64, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16,
                                          d_ff=64, tie_word_embeddings=True), batch_size=2, seq_len=16, recipe="bf16", optimizer="adamw", learning_rate=5e-2, backend="torch"))
    tr.init_weights(seed=0)
    g = GRPOTrainer(tr, GRPOLossConfig(type="ipo", kl_tau=1e-3))
    g.turn_diagnostics = True
    rng = np.random.default_rng(0)
    x = rng.integers(0, 64, (2, 16)).astype(np.int32)
    y = np.roll(x, -1, axis=1).astype(np.int32)
    y[:, :4] = -100
    y[:, 8:10] = -100       # an environment span: two turns per sample
    y[:, -1] = -100
    pos = np.tile(np.arange(16, dtype=np.int32), (2, 1))
    old = tr.token_logprobs(x, y, pos).cpu().numpy()
    adv = np.where(np.arange(2)[:, None] == 0, 1.0, -1.0).astype(np.float32) * np.ones((2, 16), np.float32)
    batch = {"inputs": x, "targets": y, "position_ids": pos, "advantages": adv, "old_logprobs": old, "seq_ids": np.tile(np.arange(2, dtype=np.int32)[:, None], (1, 16))}
    before = tr.token_logprobs(x, y, pos).cpu().numpy()
    out = None
    for _ in range(3):
        out = g.step(batch)
    after = tr.token_logprobs(x, y, pos).cpu().numpy()
    m = y != -100
    assert after[0][m[0]].mean() > before[0][m[0]].mean() and after[1][m[1]].mean() < before[1][m[1]].mean()   # rewarded up, punished down
    assert "is_masked" in out and "mismatch_kl" in out and out["turns/samples"] == 2.0 and out["turns/max_depth"] == 2.0


def test_trainer_takes_any_number_of_packed_rows():
    """A batch of 3 rows on a trainer with micro-batches of 2: padded with one empty row, run as two micro-batches, same update as the
    four-row batch built by hand."""
    from surogate_b200.grpo.config import GRPOLossConfig
    from surogate_b200.grpo.packer import Rollout, pack_rollouts
    from surogate_b200.grpo.trainer import GRPOTrainer
    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    def make():
        tr = Trainer(TrainerConfig(model=dict(architecture="Qwen3ForCausalLM", vocab_size=64, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16,
                                              d_ff=64, tie_word_embeddings=True), batch_size=2, seq_len=16, grad_accum=1, recipe="bf16", optimizer="adamw", learning_rate=1e-2,
                                   backend="torch"))
        tr.init_weights(seed=0)
        return tr, GRPOTrainer(tr, GRPOLossConfig())

    rng = np.random.default_rng(0)
    rollouts = [Rollout(list(rng.integers(1, 64, 5)), list(rng.integers(1, 64, 9)), list(-rng.random(9)), float(a), 1.0, 0, 0, {}) for a in (1.0, -1.0, 0.5)]
    variable = pack_rollouts(rollouts, 16, 0)
    assert len(variable) == 1 and variable[0].arrays()["inputs"].shape == (3, 16)
    fixed = pack_rollouts(rollouts, 16, 4)[0].arrays()
    (ta, ga), (tb, gb) = make(), make()
    out_a = ga.step(dict(variable[0].arrays()))
    assert ta.cfg.grad_accum == 2
    tb.cfg.grad_accum = 2
    out_b = gb.step(fixed)
    assert abs(out_a["loss"] - out_b["loss"]) < 1e-6 and abs(out_a["norm"] - out_b["norm"]) < 1e-6
    x = fixed["inputs"]
    assert torch.allclose(ta.logits(x[:2]), tb.logits(x[:2]), atol=1e-6)

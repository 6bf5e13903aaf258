"""Turn-resolved statistics and exploration noise of published weights."""
import numpy as np
import torch
from safetensors.torch import load_file, save_file

from surogate_b200.grpo.noise import NoiseConfig, add_noise_to_directory, read_sigma, sigma_at
from surogate_b200.grpo.turn_stats import TurnStats, turn_ids_from_mask, turn_weights


def test_turn_ids_statistics_and_weights():
    mask = np.array([1, 1, 0, 0, 1, 1, 1, 0, 1], dtype=np.int32)
    ids = turn_ids_from_mask(mask)
    assert ids.tolist() == [0, 0, -1, -1, 1, 1, 1, -1, 2]
    st = TurnStats()
    new = np.array([-1.0, -1.0, 0, 0, -0.5, -0.5, -0.5, 0, -2.0])
    old = np.array([-0.5, -0.5, 0, 0, -0.5, -0.5, -0.5, 0, -1.0])
    st.add_sample(ids, mask, new, old, token_loss=np.abs(new - old))
    st.add_sample(ids[:4], mask[:4], new[:4], old[:4], token_loss=np.abs(new - old)[:4])          # a sample that stopped after turn 0
    rows = {r["turn"]: r for r in st.rows()}
    assert rows[0]["tokens"] == 4 and rows[0]["survivors"] == 2 and rows[2]["survivors"] == 1
    assert abs(rows[0]["mean_kl"] + 0.5) < 1e-9 and rows[1]["mean_abs_kl"] == 0.0 and abs(rows[2]["mean_kl"] + 1.0) < 1e-9
    assert abs(sum(r["token_share"] for r in rows.values()) - 1) < 1e-9 and abs(sum(r["abs_kl_share"] for r in rows.values()) - 1) < 1e-9
    s = st.summary()
    assert s["turns/max_depth"] == 3 and s["turns/deep_survivor_fraction"] == 0.5 and s["turns/deep_over_shallow_abs_kl"] == 2.0
    w0, w1 = turn_weights(ids, mask, 0.0), turn_weights(ids, mask, 1.0)
    sup = mask.astype(bool)
    assert np.allclose(w0[sup], 1.0) and abs(w1.sum() - sup.sum()) < 1e-5 and np.all(w0[~sup] == 0)
    per_turn = [w1[ids == t].sum() for t in range(3)]
    assert np.allclose(per_turn, [2.0, 2.0, 2.0], atol=1e-5)            # every turn carries the same total weight


def test_noise_schedule_and_injection(tmp_path):
    cfg = NoiseConfig(enabled=True, sigma_start=1e-2, sigma_end=1e-4, stages=5)
    sig = [sigma_at(s, 100, cfg) for s in range(0, 100, 10)]
    assert sig[0] == 0.0 and sig[1] == 0.0 and abs(sig[2] - 1e-2) < 1e-12 and abs(sig[-1] - 1e-4) < 1e-12
    assert all(a >= b for a, b in zip(sig[2:], sig[3:])) and sigma_at(5, 100, NoiseConfig()) == 0.0
    tensors = {"model.layers.0.input_layernorm.weight": torch.ones(16, dtype=torch.bfloat16), "model.layers.0.self_attn.q_norm.weight": torch.ones(8),
               "model.norm.weight": torch.ones(16), "model.layers.0.mlp.up_proj.weight": torch.ones(4, 4)}
    save_file(tensors, str(tmp_path / "model.safetensors"))
    assert add_noise_to_directory(str(tmp_path), 0.05, seed=1) == 3
    out = load_file(str(tmp_path / "model.safetensors"))
    assert torch.equal(out["model.layers.0.mlp.up_proj.weight"], torch.ones(4, 4)) and out["model.layers.0.input_layernorm.weight"].dtype == torch.bfloat16
    d = (out["model.norm.weight"] - 1).abs()
    assert 0 < d.max() < 0.3 and read_sigma(str(tmp_path)) == {"sigma": 0.05, "tensors_changed": 3}
    assert add_noise_to_directory(str(tmp_path), 0.0) == 0 and read_sigma(str(tmp_path))["sigma"] == 0.0


def test_engine_side_weight_receivers_on_a_stand_in_worker(tmp_path):
    """The three receivers the rollout engine's workers mix in: files, broadcast over a group of their own, shared-memory handles."""
    import threading

    from surogate_b200.grpo.noise import add_noise_to_directory
    from surogate_b200.grpo.vllm_worker import WORKER_EXTENSIONS, ColocateWeightReceiver, FilesystemWeightReceiver, NCCLWeightReceiver, _bcast_opts

    class Model:
        def __init__(self):
            self.got = {}

        def load_weights(self, weights):
            for n, t in weights:
                self.got[n] = t.clone()

    def worker(cls):
        w = cls()
        w.model_runner = type("R", (), {"model": Model()})()
        w.device = "cpu"
        return w

    assert set(WORKER_EXTENSIONS) == {"filesystem", "nccl", "colocate"}
    named = {"model.layers.0.self_attn.q_proj.lora_A.weight": torch.randn(4, 8), "model.norm.weight": torch.ones(8)}
    save_file(named, str(tmp_path / "adapter_model.safetensors"))
    add_noise_to_directory(str(tmp_path), 0.0)
    fw = worker(FilesystemWeightReceiver)
    r = fw.update_weights_from_path(str(tmp_path))
    assert r == {"tensors": 2, "version": 1, "noise_sigma": 0.0} and torch.equal(fw.model_runner.model.got["model.norm.weight"], torch.ones(8))
    # broadcast: "trainer" = rank 0 in this thread, the engine worker = rank 1 in another
    header = [{"name": n, "shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", "")} for n, t in named.items()]
    nw = worker(NCCLWeightReceiver)
    out = {}
    th = threading.Thread(target=lambda: (nw.init_weight_group("127.0.0.1", 29795, 2, 1, "gloo"), out.update(nw.receive_weights(header))))
    th.start()
    sender = NCCLWeightReceiver()
    sender.init_weight_group("127.0.0.1", 29795, 2, 0, "gloo")
    for t in named.values():
        sender._weight_group.broadcast([t.clone()], _bcast_opts(0)).wait()
    th.join(timeout=60)
    assert out == {"tensors": 2} and all(torch.equal(nw.model_runner.model.got[n], t) for n, t in named.items())
    # handles: any (rebuild function, args) pair; on a GPU these are CUDA IPC handles
    cw = worker(ColocateWeightReceiver)
    payload = {"version": 7, "handles": {n: ((lambda x: x), (t,)) for n, t in named.items()}}
    assert cw.receive_ipc_handles(payload) == {"tensors": 2, "version": 7} and len(cw.model_runner.model.got) == 2


def test_built_in_environments_take_both_spellings_of_their_arguments(tmp_path):
    import json

    import pytest

    from surogate_b200.grpo.environments import load_environment

    env = load_environment("multihop-tools", num_examples=12, n_chains=120, min_hops=2, max_hops=4, max_turns=12, seed=1, score_rollouts=True)
    hops = {ex["info"]["hops"] for ex in env.dataset}
    assert len(env.dataset) == 12 and hops <= {2, 3, 4} and len(hops) > 1 and env.max_turns == 12
    assert {ex["info"]["hops"] for ex in load_environment("multihop-tools", num_train=5, hops=3).dataset} == {3}
    with pytest.raises(ValueError, match="unrecognised"):
        load_environment("multihop-tools", num_exampels=3)
    with pytest.raises(ValueError, match="exceeds"):
        load_environment("multihop-tools", min_hops=5, max_hops=2)
    assert len(load_environment("markdown-table-qa", max_examples=7, hf_repo="x/y", split="train", focus_types="lookup").dataset) == 7
    with pytest.raises(ValueError, match="unrecognised"):
        load_environment("markdown-table-qa", rows=3)
    data = tmp_path / "tasks.jsonl"
    data.write_text("".join(json.dumps({"input": f"task {i}", "question": f"q{i}", "answer": str(i)}) + "\n" for i in range(10)))
    a = load_environment("ruler-task", task_name="support", dataset=str(data), max_examples=4, system_prompt="be kind", seed=3, shuffle=True)
    assert len(a.dataset) == 4 and a.dataset[0]["prompt"][0]["content"].startswith("task ") and a.dataset[0]["task"] == "support" and a.system_prompt == "be kind"
    assert {ex["info"]["task_name"] for ex in a.dataset} == {"support"}
    b = load_environment("ruler-task", dataset_path=str(data), max_examples=-1)
    assert len(b.dataset) == 10 and b.dataset[2]["prompt"][0]["content"] == "q2"
    with pytest.raises(ValueError, match="unrecognised"):
        load_environment("ruler-task", dataset=str(data), taskname="x")
    with pytest.raises(ValueError, match="needs dataset_path"):
        load_environment("ruler-task")


def test_several_environments_train_together(tmp_path):
    """Prompts of two environments (one single-turn, one multi-turn) in one run: each prompt is rolled out and scored by its own
    environment, the buffer samples them by the configured ratios, episodes take their client and turn cap as arguments."""
    from surogate_b200.grpo.config import OrchestratorConfig
    from surogate_b200.grpo.config_compat import flatten_orchestrator_config
    from surogate_b200.grpo.orchestration import AsyncOrchestrator, AsyncOrchestratorConfig, make_generate_group
    from surogate_b200.grpo.orchestrator import Orchestrator
    from surogate_b200.grpo.transport.filesystem import FilesystemTransport

    flat, notes = flatten_orchestrator_config({"model": {"name": "m"}, "env": [{"id": "markdown-table-qa", "name": "tables", "args": {"num_train": 6, "num_eval": 2}},
                                                                                {"id": "multihop-tools", "args": {"num_train": 6, "num_eval": 2, "hops": 2, "max_turns": 3}}],
                                               "buffer": {"env_ratios": [0.5, 0.5]}, "rollouts_per_example": 2, "batch_size": 4})
    assert [e["name"] or e["id"] for e in flat["environments"]] == ["tables", "multihop-tools"] and not any("only the first" in n for n in notes)
    cfg = OrchestratorConfig(**{k: v for k, v in flat.items() if k in OrchestratorConfig.__dataclass_fields__})

    class Tok:
        pad_token_id = 0

        def apply_chat_template_and_encode(self, msgs, add_generation_prompt=False):
            return list(range(1, 4 + 2 * len(msgs)))

    class Client:
        def __init__(self, tag):
            self.tag, self.calls = tag, 0

        def generate(self, ctx, n, sampling):
            self.calls += 1
            return [([50 + k, 51], [-0.1, -0.2], "<answer>x</answer>" if k % 2 else "no idea") for k in range(n)]

    clients = [Client("a"), Client("b")]
    orch = Orchestrator(cfg, Tok(), clients, FilesystemTransport(str(tmp_path / "t")), lambda: 0)
    assert list(orch.envs) == ["tables", "multihop-tools"]
    orch.load_prompts()
    tasks = [p["task"] for p in orch.prompts]
    assert tasks.count("tables") == 6 and tasks.count("multihop-tools") == 6
    table_row = next(p for p in orch.prompts if p["task"] == "tables")
    hop_row = next(p for p in orch.prompts if p["task"] == "multihop-tools")
    assert orch.env_for(table_row) is orch.envs["tables"] and hasattr(orch.env_for(hop_row), "env_response") and not hasattr(orch.env_for(table_row), "env_response")
    gen = make_generate_group(orch)
    single = gen(table_row, 2, {}, 0, 0)
    multi = gen(dict(hop_row, info=dict(hop_row["info"], max_turns=1)), 2, {}, 0, 1)
    assert len(single) == 2 and all(r.completion_mask is None for r in single) and clients[0].calls == 1
    assert len(multi) == 2 and all(r.completion_mask is not None and r.meta["turns"] == 1 for r in multi) and clients[1].calls == 2   # one call per episode, on server 1
    assert orch.envs["multihop-tools"].max_turns == 3                                        # the cap travelled as an argument, the environment is untouched
    acfg = AsyncOrchestratorConfig(group_size=2, batch_size=4, sequence_len=64, rows_per_step=0, max_steps=1, max_inflight=4, workers=2,
                                   buffer={"env_ratios": [0.5, 0.5], "online_difficulty_filtering": False})
    loop = AsyncOrchestrator(acfg, orch.prompts, gen, orch.transport, lambda: 0, num_servers=2, env_names=list(orch.envs))
    assert loop.buffer.env_names == ["tables", "multihop-tools"]
    hist = loop.run()
    assert len(hist) == 1 and hist[0]["progress/total_samples"] >= 4


def test_evaluation_only_environments_score_their_own_rows(tmp_path):
    from surogate_b200.grpo.config import OrchestratorConfig
    from surogate_b200.grpo.config_compat import flatten_orchestrator_config
    from surogate_b200.grpo.orchestrator import Orchestrator

    flat, _ = flatten_orchestrator_config({"model": {"name": "m"}, "env": [{"id": "markdown-table-qa", "args": {"num_train": 4, "num_eval": 2}}],
                                           "eval": {"interval": 5, "num_examples": 3, "env": [{"id": "multihop-tools", "name": "hops", "args": {"num_train": 2, "num_eval": 5, "hops": 2}}]}})
    assert flat["eval_environments"][0]["name"] == "hops" and flat["eval_examples"] == 3
    cfg = OrchestratorConfig(**{k: v for k, v in flat.items() if k in OrchestratorConfig.__dataclass_fields__})
    orch = Orchestrator(cfg, tokenizer=None, client=None, transport=None, policy_version=lambda: 0)
    rows = orch.add_eval_environments(flat["eval_environments"], flat["eval_examples"])
    assert len(rows) == 3 and {r["task"] for r in rows} == {"hops"} and set(orch.envs) == {"markdown-table-qa", "hops"}
    assert hasattr(orch.env_for(rows[0]), "env_response") and not hasattr(orch.env_for({"task": "markdown-table-qa"}), "env_response")
    gold = rows[0]["answer"]
    assert orch.reward_fn(rows[0], [f"<answer>{gold}</answer>", "<answer>nope</answer>"]) == [1.0, 0.0]     # scored by the evaluation environment's rubric
    train_row = dict(orch.env.dataset[0], task="markdown-table-qa")
    assert len(orch.reward_fn(train_row, ["x"])) == 1


def test_episode_continues_in_a_new_sample_when_the_template_rewrites_earlier_turns(tmp_path):
    """A chat template that drops earlier reasoning breaks the token-prefix property after every turn: the episode still runs to its
    end, as one sample per turn, all with the episode's reward and advantage."""
    from surogate_b200.grpo.config import OrchestratorConfig
    from surogate_b200.grpo.orchestration import AsyncOrchestrator, AsyncOrchestratorConfig, make_generate_group
    from surogate_b200.grpo.orchestrator import Orchestrator
    from surogate_b200.grpo.transport.filesystem import FilesystemTransport

    class Env:
        max_turns = 3
        env_id = "two-step"
        dataset = [{"prompt": "go", "answer": "x"}]
        eval_dataset = []

        def initial_messages(self, row):
            return [{"role": "user", "content": row["prompt"]}]

        def setup_state(self, row):
            return {"n": 0}

        def is_completed(self, msgs, state):
            state["n"] += 1
            return state["n"] >= 3

        def env_response(self, msgs, state):
            return [{"role": "tool", "content": "ok"}]

        def score(self, row, state):
            return (1.0 if state["example"].get("good") else 0.0) + 0.0 * state["turns"], {}

    class Tok:
        """user = 10, tool = 30, assistant = header 99 + answer 20 + reasoning 21; only the LAST assistant message keeps its reasoning
        token: earlier turns are rewritten, as templates of reasoning models do."""
        pad_token_id = 0

        def apply_chat_template_and_encode(self, msgs, add_generation_prompt=False):
            ids = []
            last_assistant = max((i for i, m in enumerate(msgs) if m["role"] == "assistant"), default=-1)
            for i, m in enumerate(msgs):
                ids += {"user": [10], "tool": [30]}.get(m["role"], [99, 20, 21] if i == last_assistant else [99, 20])
            return ids + ([99] if add_generation_prompt else [])

    class Client:
        def generate(self, ctx, n, sampling):
            return [([20, 21], [-0.1, -0.2], "thinking...answer")]

    cfg = OrchestratorConfig(model="m", group_size=2, sequence_len=64)
    orch = Orchestrator(cfg, Tok(), Client(), FilesystemTransport(str(tmp_path)), lambda: 0, reward_fn=lambda r, c: [0.0] * len(c))
    orch.env = Env()
    eps = orch.multi_turn_group({"prompt": "go", "good": True}, {})
    assert len(eps) == 2 * 2 and {e[5] for e in eps} == {0, 1} and all(e[4] == 1.0 for e in eps)
    first = [e for e in eps if e[5] == 0]
    # turns 1 and 2 extend each other (one sample, the tool reply and the next header as context); after turn 2 the template drops
    # turn 1's reasoning, the prefix no longer matches, and turn 3 lives in a second sample that starts from the re-encoded conversation
    assert first[0][0] == [10, 99] and first[0][1] == [20, 21, 30, 99, 20, 21] and first[0][3] == [1, 1, 0, 0, 1, 1]
    assert first[1][0] == [10, 99, 20, 30, 99, 20, 21, 30, 99] and first[1][1] == [20, 21] and first[1][3] == [1, 1]
    gen = make_generate_group(orch)
    rollouts = gen({"prompt": "go", "good": True, "example_id": 0}, 2, {}, 0, 0)
    assert len(rollouts) == 4 and {r.meta["episode"] for r in rollouts} == {0, 1} and all(r.meta["turns"] == 3 for r in rollouts)
    # advantages are per episode: episode 0 rewarded, episode 1 not -> every sample of an episode gets the same advantage
    for r in rollouts:
        r.reward = 1.0 if r.meta["episode"] == 0 else 0.0
    loop = AsyncOrchestrator(AsyncOrchestratorConfig(group_size=2, batch_size=2, sequence_len=64, rows_per_step=0, max_steps=1, workers=1), [{"prompt": "go"}], gen,
                             orch.transport, lambda: 0)
    loop._score([rollouts])
    adv = {r.meta["episode"]: {x.advantage for x in rollouts if x.meta["episode"] == r.meta["episode"]} for r in rollouts}
    assert adv[0] == {0.5} and adv[1] == {-0.5}
    loop.pool.shutdown(wait=False)

"""The orchestrator's building blocks without a server: buffer pools, scheduler staleness rules, filters, advantages, depth budget."""
import math

import numpy as np

from surogate_b200.grpo.orchestration import (BufferConfig, DepthObservation, ExampleBuffer, GibberishFilter, RepetitionFilter, RolloutDepthController,
                                              RolloutScheduler, SchedulerConfig, apply_filters, compute_advantages, make_filters)
from surogate_b200.grpo.packer import Rollout


def _rollout(reward=0.0, n=8, ex=0, task="default", lp=-1.0, ids=None):
    ids = list(ids) if ids is not None else list(range(n))
    return Rollout(prompt_ids=[1, 2, 3], completion_ids=ids, logprobs=[lp] * len(ids), reward=reward, meta={"example_id": ex, "task": task})


def test_buffer_moves_solved_and_hopeless_prompts_out_of_the_sampling_pool_and_round_trips(tmp_path):
    ex = [{"prompt": f"q{i}", "task": "math" if i % 2 else "code"} for i in range(20)]
    buf = ExampleBuffer(ex, BufferConfig(seed=1, easy_threshold=1.0, hard_threshold=0.0, min_normal=4, easy_fraction=0.5, hard_fraction=0.5), ["code", "math"])
    assert buf.count("normal") == 20 and abs(sum(buf.env_probs.values()) - 1) < 1e-9
    drawn = buf.sample_examples(50)
    assert {d["task"] for d in drawn} == {"code", "math"}
    # ids 0..5 always solved, 6..11 never, 12 mixed
    groups = [[_rollout(1.0, ex=i, task=ex[i]["task"]) for _ in range(4)] for i in range(6)]
    groups += [[_rollout(0.0, ex=i, task=ex[i]["task"]) for _ in range(4)] for i in range(6, 12)]
    groups += [[_rollout(float(k % 2), ex=12, task=ex[12]["task"]) for k in range(4)]]
    buf.update(groups)
    assert buf.count("easy") == 6 and buf.count("hard") == 6 and buf.count("normal") == 8
    assert buf.step["filtered_groups"] == 12 and len(buf.rollouts) == 4          # only the mixed group carries signal
    assert all(d["example_id"] >= 12 for d in buf.sample_examples(40))
    assert len(buf.sample_rollouts(3)) == 3 and len(buf.rollouts) == 1
    buf.save(str(tmp_path))
    fresh = ExampleBuffer(list(reversed(ex)), BufferConfig(seed=2, easy_threshold=1.0, hard_threshold=0.0), ["code", "math"])
    # ids differ after re-ordering; membership follows the prompt hash
    assert fresh.load(str(tmp_path)) == 12 and fresh.count("easy") == 6 and fresh.count("hard") == 6
    # recycling: drain normal below the floor
    for env in buf.env_names:
        for i in list(buf.pools["normal"][env])[:-1]:
            buf.pools["hard"][env][i] = buf.pools["normal"][env].pop(i)
    before = buf.count("normal")
    buf.sample_examples(1)
    assert buf.count("normal") > before and buf.step["recycled"] > 0
    m = buf.metrics()
    assert abs(m["buffer/easy"] + m["buffer/normal"] + m["buffer/hard"] - 1) < 1e-9


def test_scheduler_bounds_inflight_requests_and_staleness():
    ex = [{"prompt": f"q{i}", "example_id": i} for i in range(100)]
    buf = ExampleBuffer(ex, BufferConfig(seed=0))
    pending, cancelled = {}, []

    def submit(example, version, server):
        h = len(pending)
        pending[h] = dict(example=example, version=version, server=server, done=False)
        return h

    def poll(h):
        p = pending[h]
        return [_rollout(float(k % 2), ex=p["example"]["example_id"]) for k in range(4)] if p["done"] else None

    s = RolloutScheduler(SchedulerConfig(batch_size=8, group_size=4, max_inflight=6, max_async_level=1, max_off_policy_steps=1), buf, submit, poll,
                         cancel=cancelled.append, num_servers=2)
    assert s.fill(step=0) == 6 and len(s.inflight) == 6 and s.fill(step=0) == 0
    assert {p["server"] for p in pending.values()} == {0, 1}
    assert not s.may_issue(step=2) and s.may_issue(step=1)               # generation may not run more than one version ahead
    for h in (0, 1, 2):
        pending[h]["done"] = True
    assert s.collect() == 3 and s.batch_ready()
    batch = s.take_batch()
    assert len(batch) == 2 and all(r.policy_version == 0 and r.meta["off_policy_level"] == 0 for g in batch for r in g)
    assert len(s.ready) == 1                                             # whole groups only; the third waits for the next batch
    # two policy updates later the three requests still in flight are too stale: cancelled and re-queued
    assert s.on_policy_update(1) == 0
    assert s.on_policy_update(2) == 3 and len(cancelled) == 3 and len(s.requeued) == 3
    s.fill(step=2)
    assert [p["example"]["example_id"] for h, p in pending.items() if h >= 6][:3] == [pending[h]["example"]["example_id"] for h in (3, 4, 5)]
    pending[6]["done"] = True
    s.collect()
    batch = s.take_batch()
    assert batch[0][0].meta["off_policy_level"] == 2                     # the group that waited since version 0
    m = s.metrics()
    assert m["scheduler/cancelled"] == 3 and m["scheduler/off_policy_max"] == 2
    # token batching and the depth cap
    s2 = RolloutScheduler(SchedulerConfig(token_batch_size=40, group_size=4, max_inflight=2), buf, submit, poll)
    s2.set_depth_cap(3)
    capped = s2._example_with_cap({"prompt": "x", "info": {"max_turns": 10}})
    assert capped["info"]["max_turns"] == 3 and s2.uses_token_batching and s2.batch_target == 40


def test_filters_flag_noise_and_loops_and_mask_them_out():
    vocab = 50000
    g = GibberishFilter(vocab)
    assert g.check(_rollout(n=64, lp=-math.log(vocab) + 0.5)).detected and not g.check(_rollout(n=64, lp=-1.5)).detected
    assert not g.check(_rollout(n=4, lp=-20.0)).detected                  # too short to judge
    r = RepetitionFilter(ngram=4, max_consecutive=5)
    loop = [7, 8, 9, 10] * 30
    assert r.check(_rollout(ids=loop)).detected and not r.check(_rollout(ids=list(range(200)))).detected
    fs = make_filters([{"type": "gibberish"}, {"type": "repetition", "ngram": 4, "max_consecutive": 5}], vocab)
    ros = [_rollout(n=64, lp=-11.0), _rollout(ids=loop), _rollout(n=64, lp=-0.5)]
    stats = apply_filters(fs, ros)
    assert abs(stats["filter/gibberish"] - 1 / 3) < 1e-9 and abs(stats["filter/repetition"] - 1 / 3) < 1e-9
    assert sum(ros[0].completion_mask) == 0 and ros[1].meta["filtered"] == "repetition" and ros[2].completion_mask is None


def test_advantages():
    rewards = [1, 0, 0, 1, 2, 2, 2, 2]
    lens = [10, 30, 10, 10, 5, 5, 5, 5]
    a = compute_advantages(rewards, lens, 4)
    assert np.allclose(a, [0.5, -0.5, -0.5, 0.5, 0, 0, 0, 0])
    lw = compute_advantages(rewards, lens, 4, length_weighted_mean=True)
    assert np.allclose(lw[:4], np.array([1, 0, 0, 1]) - (10 + 10) / 60)
    s = compute_advantages(rewards, lens, 4, kind="std")
    assert abs(s[0] - 0.5 / (0.5 + 1e-4)) < 1e-6 and s[4] == 0.0
    assert compute_advantages(rewards, lens, 4, custom=lambda inp: type("O", (), {"advantages": inp.rewards * 2})()) == [2, 0, 0, 2, 4, 4, 4, 4]


def test_depth_budget_follows_the_depths_that_earned_reward():
    c = RolloutDepthController(quantile=0.9, headroom=1.25, probe_every=4, min_observations=20, max_cap=40)
    assert c.cap_for_step(1) == 40                                        # nothing known yet: the configured maximum
    obs = [DepthObservation(depth=d, reward=1.0) for d in [3, 4, 4, 5, 5, 5, 6, 6, 7, 8] * 3] + [DepthObservation(depth=35, reward=0.0) for _ in range(10)]
    c.observe(1, obs)
    assert c.cap is not None and 8 <= c.cap <= 10                         # deep, unrewarded episodes do not raise the budget
    assert c.cap_for_step(2) == c.cap and c.cap_for_step(4) == 40 and c.is_probe_step(8)
    c.observe(4, [DepthObservation(depth=20, reward=1.0) for _ in range(200)])   # the probe step finds that deeper episodes now pay
    assert c.cap >= 20 and c.metrics()["depth/cap"] == c.cap
    off = RolloutDepthController(enabled=False, max_cap=12)
    assert off.cap_for_step(3) == 12 and not off.is_probe_step(0)


def test_async_loop_ships_batches_with_signal_and_resumes_from_its_checkpoint(tmp_path):
    import threading

    from surogate_b200.grpo.orchestration import AsyncOrchestrator, AsyncOrchestratorConfig
    from surogate_b200.grpo.transport.filesystem import FilesystemTransport

    examples = [{"prompt": f"q{i}", "kind": "solved" if i < 4 else "mixed"} for i in range(12)]
    calls = {"n": 0}
    lock = threading.Lock()

    def generate_group(example, n, sampling, version, server):
        with lock:
            calls["n"] += 1
        out = []
        for k in range(n):
            reward = 1.0 if example["kind"] == "solved" else float(k % 2)
            out.append(Rollout(prompt_ids=[1, 2], completion_ids=list(range(3, 3 + 6 + k)), logprobs=[-0.5] * (6 + k), reward=reward, meta={"turns": 1 + k % 3}))
        return out

    version = {"v": 0}
    cfg = AsyncOrchestratorConfig(group_size=4, batch_size=8, sequence_len=64, rows_per_step=4, max_steps=3, max_inflight=4, max_async_level=1, workers=4,
                                  buffer={"easy_threshold": 1.0, "seed": 3}, checkpoint_dir=str(tmp_path / "ckpt"), checkpoint_every=1,
                                  depth={"enabled": True, "min_observations": 4, "probe_every": 2, "max_cap": 9}, filters=[{"type": "repetition", "ngram": 2, "min_tokens": 1000}])
    tr = FilesystemTransport(str(tmp_path / "rollouts"))
    seen = []

    def on_step(m):
        seen.append(m)
        version["v"] += 1     # the trainer consumed the batch and published

    orch = AsyncOrchestrator(cfg, examples, generate_group, tr, lambda: version["v"], on_step=on_step)
    hist = orch.run()
    assert len(hist) == 3 and len(seen) == 3
    for step in range(3):
        arrays, meta = tr.receive(step, timeout_s=1)
        assert arrays["inputs"].shape == (4, 64) and meta["n_samples"] == 8
        adv = arrays["advantages"][arrays["targets"] != -100]
        assert np.abs(adv).max() > 0 and set(np.round(np.unique(adv), 3)) == {-0.5, 0.5}     # only mixed-reward groups were shipped
    assert orch.buffer.count("easy") >= 1 and hist[-1]["buffer/filtered_groups"] >= 0
    assert hist[-1]["depth/cap"] >= 2 and hist[-1]["scheduler/off_policy_max"] <= cfg.max_off_policy_steps
    # resume: progress and pools come back
    again = AsyncOrchestrator(AsyncOrchestratorConfig(**{**cfg.__dict__, "max_steps": 4}), examples, generate_group, tr, lambda: 10)
    assert again.resume() == 3 and again.buffer.count("easy") == orch.buffer.count("easy")
    again.run()
    assert tr.ready(3)


def test_gpu_sets_are_validated_and_a_failing_component_takes_the_run_down(tmp_path):
    import sys
    import time

    import pytest

    from surogate_b200.grpo.runners import Component, Supervisor, check_disjoint, check_topology, parse_gpu_ids, plan_colocate, plan_split

    assert parse_gpu_ids("0-2,5") == [0, 1, 2, 5] and parse_gpu_ids("") == []
    with pytest.raises(ValueError, match="twice"):
        parse_gpu_ids("0,0")
    with pytest.raises(ValueError, match="both"):
        check_disjoint(("trainer", [0, 1]), ("rollout engine", [1, 2]))
    with pytest.raises(ValueError, match="needs 4"):
        check_topology("rollout engine", [4, 5], tensor_parallel=2, data_parallel=2)
    comps = plan_split("t.yaml", "i.yaml", "o.yaml", "0-3", "4-7", tensor_parallel=2, data_parallel=2, max_steps=5)
    by = {c.name: c for c in comps}
    assert by["trainer"].env["CUDA_VISIBLE_DEVICES"] == "0,1,2,3" and "--nproc-per-node=4" in by["trainer"].argv and "127.0.0.1" in by["trainer"].argv
    assert by["rollout engine"].env["CUDA_VISIBLE_DEVICES"] == "4,5,6,7" and by["orchestrator"].env["CUDA_VISIBLE_DEVICES"] == ""
    with pytest.raises(ValueError, match="judge"):
        plan_split("t", "i", "o", "0", "1", judge_cfg="j.yaml")
    co = plan_colocate("t.yaml", "i.yaml", "o.yaml", "0,1", engine_memory_fraction=0.4)
    assert co[0].env["SUROGATE_ENGINE_MEMORY_FRACTION"] == "0.4" and co[1].env["SUROGATE_GRPO_COLOCATE"] == "1"
    # supervision with stand-in processes: the engine sleeps, the orchestrator fails -> everything stops, its code is returned
    marker = tmp_path / "engine_stopped"
    engine = Component("rollout engine", [sys.executable, "-c", "import signal,sys,time,pathlib\n"
                                          f"signal.signal(signal.SIGTERM, lambda *a: (pathlib.Path(r'{marker}').write_text('x'), sys.exit(0)))\n"
                                          "time.sleep(60)"])
    bad = Component("orchestrator", [sys.executable, "-c", "import sys,time; time.sleep(0.3); sys.exit(7)"])
    log = []
    t0 = time.time()
    rc = Supervisor([engine, bad], grace_s=5, poll_s=0.05, log=log.append).run(timeout_s=30)
    assert rc == 7 and time.time() - t0 < 20 and marker.exists() and engine.proc.poll() is not None
    # trainer finishing ends the run with 0 and stops the engine
    engine2 = Component("rollout engine", [sys.executable, "-c", "import time; time.sleep(60)"])
    trainer = Component("trainer", [sys.executable, "-c", "print('done')"], ends_run_on_success=True)
    assert Supervisor([engine2, trainer], grace_s=5, poll_s=0.05, log=log.append).run(timeout_s=30) == 0 and engine2.proc.poll() is not None


def test_cli_dry_run_lists_the_three_components(tmp_path, capsys):
    import json as _json

    from surogate_b200.cli.main import cli_main

    for n in ("t", "i", "o"):
        (tmp_path / f"{n}.yaml").write_text("tensor_parallel_size: 1\n")
    rc = cli_main(["grpo-train", "--train", str(tmp_path / "t.yaml"), "--infer", str(tmp_path / "i.yaml"), "--orch", str(tmp_path / "o.yaml"),
                   "--trainer-gpus", "0", "--vllm-gpus", "1", "--dry-run"])
    lines = [_json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert rc == 0 and [l["name"] for l in lines] == ["rollout engine", "trainer", "orchestrator"]
    rc = cli_main(["grpo-colocate", "--train", str(tmp_path / "t.yaml"), "--infer", str(tmp_path / "i.yaml"), "--orch", str(tmp_path / "o.yaml"), "--dry-run"])
    assert rc == 0 and "grpo-infer" in capsys.readouterr().out


def test_async_loop_runs_on_the_parts_of_a_configured_orchestrator(tmp_path):
    """``make_generate_group`` + ``async_config_from``: the asynchronous loop driven by the same tokenizer / client / reward objects
    the synchronous orchestrator uses (a fake client and tokenizer stand in for the server)."""
    from surogate_b200.grpo.config import OrchestratorConfig
    from surogate_b200.grpo.orchestration import AsyncOrchestrator, async_config_from, make_generate_group
    from surogate_b200.grpo.orchestrator import Orchestrator
    from surogate_b200.grpo.transport.filesystem import FilesystemTransport

    class Tok:
        pad_token_id, vocab_size = 0, 100

        def apply_chat_template_and_encode(self, messages, add_generation_prompt=True):
            return [1] + [2 + (ord(c) % 50) for c in messages[-1]["content"]][:6]

    class Client:
        def __init__(self):
            self.calls = 0

        def generate(self, prompt_ids, n, sampling):
            self.calls += 1
            return [([10 + k, 11, 12], [-0.1, -0.2, -0.3], "yes" if k % 2 else "no") for k in range(n)]

    cfg = OrchestratorConfig(model="m", group_size=4, prompts_per_step=2, sequence_len=32, rows_per_step=2, max_steps=2, max_async_level=4, reward="exact_match")
    clients = [Client(), Client()]
    tr = FilesystemTransport(str(tmp_path))
    orch = Orchestrator(cfg, Tok(), clients, tr, lambda: 0, reward_fn=lambda row, texts: [1.0 if t == row["answer"] else 0.0 for t in texts])
    orch.load_prompts([{"prompt": f"q{i}", "answer": "yes"} for i in range(6)])
    acfg = async_config_from(cfg, {"max_inflight": 4, "workers": 2, "filters": [{"type": "repetition"}]}, vocab_size=100)
    assert acfg.batch_size == 8 and acfg.sampling["max_tokens"] == cfg.max_tokens and acfg.filters
    loop = AsyncOrchestrator(acfg, orch.prompts, make_generate_group(orch), tr, lambda: 0, num_servers=2)
    hist = loop.run()
    assert len(hist) == 2 and clients[0].calls > 0 and clients[1].calls > 0          # both servers were used
    arrays, meta = tr.receive(1, timeout_s=1)
    adv = arrays["advantages"][arrays["targets"] != -100]
    assert meta["n_samples"] == 8 and set(np.round(np.unique(adv), 3)) == {-0.5, 0.5}


def test_periodic_evaluation_reports_pass_at_k_without_feeding_the_trainer(tmp_path):
    from surogate_b200.grpo.orchestration import AsyncOrchestrator, AsyncOrchestratorConfig, evaluate_policy, pass_at_k
    from surogate_b200.grpo.transport.filesystem import FilesystemTransport

    assert pass_at_k(4, 0, 2) == 0.0 and pass_at_k(4, 4, 1) == 1.0 and abs(pass_at_k(4, 1, 1) - 0.25) < 1e-12 and abs(pass_at_k(4, 1, 2) - 0.5) < 1e-12
    assert pass_at_k(2, 1, 8) == 1.0            # k is capped at n

    def generate_group(example, n, sampling, version, server):
        solved = {"always": n, "half": n // 2, "never": 0}[example["kind"]]
        return [_rollout(1.0 if k < solved else 0.0, n=5 + k) for k in range(n)]

    held_out = [{"prompt": "a", "kind": "always"}, {"prompt": "b", "kind": "half"}, {"prompt": "c", "kind": "never"}]
    m = evaluate_policy(held_out, generate_group, 4, {}, ks=(1, 2))
    assert abs(m["eval/mean_reward"] - 0.5) < 1e-12 and abs(m["eval/pass@1"] - 0.5) < 1e-12 and abs(m["eval/unsolved_fraction"] - 1 / 3) < 1e-12
    assert abs(m["eval/pass@2"] - (1 + (1 - 1 / 6) + 0) / 3) < 1e-12
    train = [{"prompt": f"q{i}", "kind": "half"} for i in range(6)]
    cfg = AsyncOrchestratorConfig(group_size=4, batch_size=8, sequence_len=64, rows_per_step=4, max_steps=2, max_inflight=4, workers=2, eval_every=2, eval_samples=4,
                                  eval_ks=(1, 2))
    tr = FilesystemTransport(str(tmp_path))
    hist = AsyncOrchestrator(cfg, train, generate_group, tr, lambda: 0, eval_examples=held_out).run()
    assert "eval/pass@1" not in hist[0] and abs(hist[1]["eval/pass@1"] - 0.5) < 1e-12
    _, meta = tr.receive(1, timeout_s=1)
    assert meta["n_samples"] == 8              # the evaluation rollouts did not join the batch


def test_rate_limit_validation_rollouts_and_metrics_file(tmp_path):
    import json

    from surogate_b200.grpo.orchestration import AsyncOrchestrator, AsyncOrchestratorConfig
    from surogate_b200.grpo.transport.filesystem import FilesystemTransport

    # token bucket: 30 requests per minute = one every two seconds, the first one at once
    ex = [{"prompt": f"q{i}", "example_id": i} for i in range(50)]
    buf = ExampleBuffer(ex, BufferConfig(seed=0))
    issued = []
    s = RolloutScheduler(SchedulerConfig(batch_size=8, group_size=4, max_inflight=100, max_async_level=4, tasks_per_minute=30.0), buf,
                         lambda e, v, srv: issued.append(e) or len(issued), lambda h: None)
    now = [100.0]
    s.clock = lambda: now[0]
    assert s.fill(0) == 1 and s.fill(0) == 0
    now[0] += 1.9
    assert s.fill(0) == 0
    now[0] += 0.2
    assert s.fill(0) == 1
    now[0] += 600.0                                # a long pause saves up at most one minute's worth
    assert s.fill(0) == 30
    unlimited = RolloutScheduler(SchedulerConfig(batch_size=8, group_size=4, max_inflight=7, max_async_level=4), buf, lambda e, v, srv: 1, lambda h: None)
    assert unlimited.fill(0) == 7

    calls = {"n": 0}

    def generate_group(example, n, sampling, version, server):
        calls["n"] += 1
        return [_rollout(float(k % 2), n=5 + k) for k in range(n)]

    train = [{"prompt": f"q{i}"} for i in range(6)]
    cfg = AsyncOrchestratorConfig(group_size=4, batch_size=8, sequence_len=64, rows_per_step=0, max_steps=2, max_inflight=4, workers=2, val_every=2, val_examples=3,
                                  val_samples=2, metrics_file=str(tmp_path / "m" / "metrics.jsonl"))
    tr = FilesystemTransport(str(tmp_path / "t"))
    hist = AsyncOrchestrator(cfg, train, generate_group, tr, lambda: 0).run()
    assert "val/mean_reward" not in hist[0] and abs(hist[1]["val/mean_reward"] - 0.5) < 1e-12 and hist[1]["val/examples"] == 3.0
    rows = [json.loads(l) for l in open(tmp_path / "m" / "metrics.jsonl")]
    assert len(rows) == 2 and rows[1]["val/mean_reward"] == 0.5 and "reward/mean" in rows[0]
    batch, meta = tr.receive(1, timeout_s=1)
    assert meta["n_samples"] == 8 and batch["inputs"].shape[0] >= 1      # validation rollouts did not join the batch; rows as needed


def test_supervisor_reaps_workers_that_left_their_process_group(tmp_path):
    """A component starts a worker in a session of its own and dies: with the subreaper flag the worker re-parents to the
    supervisor's process and the final walk ends it (a ``killpg`` of the component's group alone would miss it)."""
    import os
    import subprocess
    import sys
    import textwrap
    import time

    import psutil

    script = textwrap.dedent(f"""
        import os, sys, time
        sys.path.insert(0, {os.getcwd()!r})
        from surogate_b200.grpo.runners import Component, Supervisor
        worker = "import time, os; open({str(tmp_path / 'worker.pid')!r}, 'w').write(str(os.getpid())); time.sleep(300)"
        comp = ("import subprocess, sys, time; subprocess.Popen([sys.executable, '-c', " + repr(worker) + "], start_new_session=True); time.sleep(1.0); sys.exit(3)")
        sup = Supervisor([Component("engine", [sys.executable, "-c", comp], {{}})], grace_s=2.0, poll_s=0.05, log=lambda m: print(m, flush=True), reap=True)
        rc = sup.run(timeout_s=30)
        print("rc", rc, flush=True)
    """)
    p = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=120)
    assert "rc 3" in p.stdout, p.stdout + p.stderr
    pid = int(open(tmp_path / "worker.pid").read())
    deadline = time.time() + 5
    while psutil.pid_exists(pid) and time.time() < deadline:
        time.sleep(0.05)
    gone = not psutil.pid_exists(pid) or psutil.Process(pid).status() == psutil.STATUS_ZOMBIE
    if not gone:
        os.kill(pid, 9)
    assert gone and "reaped 1 leftover" in p.stdout, p.stdout

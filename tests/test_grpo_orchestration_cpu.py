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

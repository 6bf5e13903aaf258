"""LLM-judge group rewards (``grpo/ruler.py``) against a local judge stand-in: request shape, score parsing, retries, modes, the
orchestrator hooks for single-turn groups and multi-turn episodes."""
import json
import threading
from http.server import BaseHTTPRequestHandler, HTTPServer

import pytest

from surogate_b200.grpo.ruler import JudgePool, RulerConfig, RulerJudgeError, RulerScorer, build_ruler, common_prefix_len, parse_scores


class _Judge:
    """Scores a trajectory by the number in its last assistant message (divided by 10); scripted failures come first."""

    def __init__(self, script=()):
        self.script, self.bodies, self.paths = list(script), [], []
        judge = self

        class H(BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def do_GET(self):
                judge.paths.append(self.path)
                self._send(200, {"data": [{"id": "judge"}]})

            def do_POST(self):
                body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
                judge.bodies.append(body)
                judge.paths.append(self.path)
                action = judge.script.pop(0) if judge.script else "ok"
                if action == "500":
                    return self._send(500, {})
                if action == "garbage":
                    return self._send(200, {"choices": [{"message": {"content": "I think they are all fine."}}], "usage": {"prompt_tokens": 10, "completion_tokens": 5}})
                user = body["messages"][1]["content"]
                import re

                scores = []
                for m in re.finditer(r'<trajectory id="(\d+)">\n(.*?)\n</trajectory>', user, re.S):
                    last = json.loads(m.group(2).strip().splitlines()[-1])["content"]
                    scores.append({"trajectory_id": m.group(1), "explanation": "by the number", "score": float(re.sub(r"\D", "", last) or 0) / 10.0})
                scores.reverse()  # any order is fine
                self._send(200, {"choices": [{"message": {"content": "```json\n" + json.dumps({"scores": scores}) + "\n```"}}], "usage": {"prompt_tokens": 100, "completion_tokens": 20}})

            def _send(self, code, obj):
                data = json.dumps(obj).encode()
                self.send_response(code)
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

        self.srv = HTTPServer(("127.0.0.1", 0), H)
        threading.Thread(target=self.srv.serve_forever, daemon=True).start()
        self.url = f"http://127.0.0.1:{self.srv.server_port}/v1"

    def close(self):
        self.srv.shutdown()


def _traj(answer):
    return [{"role": "system", "content": "be exact"}, {"role": "user", "content": "what is 2+2"}, {"role": "assistant", "content": answer}]


def test_score_parsing_and_prefix():
    assert parse_scores('{"scores": [{"trajectory_id": "2", "score": 0.25}, {"trajectory_id": "trajectory-1", "score": 1.7}]}', 2) == [1.0, 0.25]
    assert parse_scores('noise {"scores": [0.1, 0.9]} tail', 2) == [0.1, 0.9]
    for bad, n in (("nothing here", 2), ('{"scores": [0.1]}', 2), ('{"scores": [{"trajectory_id": "1", "score": 0.5}]}', 2), ('{"other": 1}', 1),
                   ('{"scores": [{"trajectory_id": "1"}]}', 1)):
        with pytest.raises(ValueError):
            parse_scores(bad, n)
    assert common_prefix_len([_traj("4"), _traj("5")]) == 2 and common_prefix_len([_traj("4"), _traj("4")]) == 3 and common_prefix_len([]) == 0
    with pytest.raises(ValueError):
        RulerConfig(mode="multiply")
    with pytest.raises(ValueError):
        RulerConfig(enabled=True)
    with pytest.raises(ValueError):
        RulerConfig.from_dict({"enabled": False, "jugde": {}})
    assert build_ruler({"enabled": False}) is None and build_ruler(None) is None


def test_group_scoring_modes_retries_and_cost():
    j = _Judge(script=["500", "garbage"])
    try:
        cfg = RulerConfig(enabled=True, mode="add", judge_model="judge", judge={"base_url": [j.url], "api_key_var": None}, weight=2.0, max_retries_on_parse_error=2,
                          cost={"input_per_million": 1.0, "output_per_million": 4.0}, sampling={"max_tokens": 256})
        s = RulerScorer(cfg, JudgePool.from_config(cfg))
        s.pool.wait_for_ready(timeout_s=5)
        assert "/v1/models" in j.paths
        out, metrics = s.apply([_traj("7"), _traj("3"), _traj("10")], [1.0, 0.0, 0.5])
        assert out == [1.0 + 1.4, 0.0 + 0.6, 0.5 + 2.0] and metrics["ruler/failed"] == 0.0 and abs(metrics["ruler/score_mean"] - 2.0 / 3) < 1e-9
        assert len(j.bodies) == 3                                   # one transport retry, one parse retry, then the answer
        body = j.bodies[-1]
        assert body["model"] == "judge" and body["max_tokens"] == 256 and body["temperature"] == 0.0
        user = body["messages"][1]["content"]
        assert user.count("be exact") == 1 and user.count("<trajectory id=") == 3 and "<context>" in user   # the shared beginning is sent once
        m = s.metrics()
        assert m["ruler/groups"] == 1 and m["ruler/parse_retries"] == 1 and m["ruler/failures"] == 0 and m["ruler/input_tokens"] == 110
        assert abs(m["ruler/cost"] - (110 * 1.0 + 25 * 4.0) / 1e6) < 1e-12
        s.cfg.mode = "replace"
        assert s.apply([_traj("7"), _traj("3")], [9.0, 9.0])[0] == [1.4, 0.6]
        s.cfg.mode = "metric"
        assert s.apply([_traj("7"), _traj("3")], [9.0, 8.0])[0] == [9.0, 8.0]
        assert s.score_group([_traj("7")]) == [0.5] and s.score_group([]) == []
        # a judge that never produces parsable scores: swallowed (zeros in replace mode, counted) or raised
        j.script += ["garbage"] * 3
        s.cfg.mode = "replace"
        out, metrics = s.apply([_traj("7"), _traj("3")], [1.0, 1.0])
        assert out == [0.0, 0.0] and metrics == {"ruler/failed": 1.0} and s.metrics()["ruler/failures"] == 1
        j.script += ["garbage"] * 3
        s.cfg.swallow_exceptions = False
        with pytest.raises(RulerJudgeError):
            s.apply([_traj("7"), _traj("3")], [1.0, 1.0])
    finally:
        j.close()
    dead = JudgePool(["http://127.0.0.1:9/v1"], max_retries=1, timeout_s=0.5)
    with pytest.raises(RulerJudgeError, match="unreachable"):
        dead.chat({"model": "x", "messages": []})


def test_pool_round_robin_over_endpoints():
    a, b = _Judge(), _Judge()
    try:
        pool = JudgePool([a.url, b.url], max_concurrent=2)
        s = RulerScorer(RulerConfig(enabled=True, judge_model="judge"), pool)
        for _ in range(4):
            s.score_group([_traj("1"), _traj("2")])
        assert len(a.bodies) == 2 and len(b.bodies) == 2 and pool.requests == 4
    finally:
        a.close()
        b.close()


def test_orchestrator_uses_the_judge_for_single_and_multi_turn_groups():
    from surogate_b200.grpo.config import OrchestratorConfig
    from surogate_b200.grpo.orchestrator import Orchestrator

    j = _Judge()
    try:
        ruler = {"enabled": True, "mode": "add", "judge_model": "judge", "judge": {"base_url": j.url, "api_key_var": None}, "weight": 1.0}
        cfg = OrchestratorConfig(model="m", group_size=2, ruler=ruler)
        orch = Orchestrator(cfg, tokenizer=None, client=None, transport=None, policy_version=lambda: 0, reward_fn=lambda row, cs: [1.0 if c == "4" else 0.0 for c in cs])
        assert orch.judge is not None
        assert orch.reward_fn({"prompt": "what is 2+2"}, ["4", "9"]) == [1.0 + 0.4, 0.0 + 0.9]

        class Env:
            max_turns = 2

            def initial_messages(self, row):
                return [{"role": "user", "content": row["prompt"]}]

            def setup_state(self, row):
                return {}

            def is_completed(self, msgs, state):
                return True

            def env_response(self, msgs, state):
                return []

            def score(self, row, state):
                return 0.25, {}

        class Tok:
            def apply_chat_template_and_encode(self, msgs, add_generation_prompt=False):
                return [1, 2, 3]

        class Client:
            n = 0

            def generate(self, ctx, n, sampling):
                Client.n += 1
                return [([7, 8], [-0.1, -0.2], str(Client.n * 3))]

        orch.env, orch.tok, orch.client = Env(), Tok(), Client()
        eps = orch.multi_turn_group({"prompt": "count"}, {})
        assert [round(e[4], 6) for e in eps] == [0.25 + 0.3, 0.25 + 0.6] and all(e[1] == [7, 8] for e in eps)
    finally:
        j.close()


def test_teacher_scores_travel_from_the_server_to_the_packed_batch():
    """A served teacher's ``prompt_logprobs`` become per-token ``teacher_logprobs`` of the rollouts, aligned with the targets in the
    packed batch, and reach the ``ipo`` objective's teacher term."""
    import numpy as np
    import torch

    from surogate_b200.grpo.config_compat import flatten_orchestrator_config
    from surogate_b200.grpo.loss import ipo_token_weights
    from surogate_b200.grpo.packer import Rollout, pack_rollouts
    from surogate_b200.grpo.teacher import TeacherScorer

    seen = []

    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            seen.append(body)
            ids = body["prompt"]
            # position t: the teacher's log-prob of token t is -(t + 1) / 10; a second, wrong candidate is listed too
            entries = [None] + [{str(tok): {"logprob": -(t + 1) / 10.0}, "99999": {"logprob": -9.0}} for t, tok in enumerate(ids[1:], 1)]
            data = json.dumps({"choices": [{"prompt_logprobs": entries}]}).encode()
            self.send_response(200)
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

    srv = HTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        flat, notes = flatten_orchestrator_config({"model": {"name": "m"}, "teacher_model": {"model": {"name": "big"}, "client": {"base_url": [f"http://127.0.0.1:{srv.server_port}/v1"],
                                                                                                                   "api_key_var": None}}})
        assert not any("teacher" in n for n in notes)
        t = TeacherScorer.from_config(flat["teacher"])
        rs = [Rollout([1, 2, 3], [4, 5], [-0.5, -0.6], 1.0), Rollout([7], [8, 9, 10], [-0.1, -0.2, -0.3], -1.0)]
        t.score(rs)
    finally:
        srv.shutdown()
    assert seen[0]["model"] == "big" and seen[0]["prompt"] == [1, 2, 3, 4, 5] and seen[0]["prompt_logprobs"] == 1
    assert np.allclose(rs[0].teacher_logprobs, [-0.4, -0.5]) and np.allclose(rs[1].teacher_logprobs, [-0.2, -0.3, -0.4]) and t.tokens_scored == 5
    batch = pack_rollouts(rs, 8, 0)[0].arrays()
    y, teach, old = batch["targets"], batch["teacher_logprobs"], batch["old_logprobs"]
    assert teach.shape == y.shape and ((teach != 0) == (y != -100)).all()
    row = int(np.argmax((batch["inputs"][:, 0] == 1)))
    assert np.allclose(teach[row][y[row] != -100], [-0.4, -0.5]) and np.allclose(old[row][y[row] != -100], [-0.5, -0.6])
    assert "teacher_logprobs" not in pack_rollouts([Rollout([1], [2], [-0.1])], 8, 0)[0].arrays()
    # the teacher term moves the weights: a token the teacher likes more than the policy gets a larger multiplier
    logp = torch.from_numpy(old)
    m = torch.from_numpy((y != -100).astype(np.float32))
    adv = torch.from_numpy(batch["advantages"])
    _, w0, _ = ipo_token_weights(logp, logp, adv, m, kl_tau=0.0)
    _, w1, met = ipo_token_weights(logp, logp, adv, m, teacher_logp=torch.from_numpy(teach), teacher_tau=1.0, kl_tau=0.0)
    assert torch.allclose((w1 - w0)[m.bool()], ((torch.from_numpy(teach) - logp) / m.sum())[m.bool()], atol=1e-7) and "teacher_kl" in met
    with pytest.raises(ValueError):
        TeacherScorer.from_config({"model": "x"})
    assert TeacherScorer.from_config({}) is None

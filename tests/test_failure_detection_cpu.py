"""Failure detection without a GPU fault: a rank that raises, a rank that vanishes, a truncated checkpoint shard."""
import json
import os
import subprocess
import sys
import time

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(args, port, nproc=2, timeout=90):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1", WORLD_SIZE=str(nproc))
    procs = []
    for r in range(nproc):
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "wd_worker.py"), json.dumps(args)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = {}
    t0 = time.time()
    for r, p in enumerate(procs):
        try:
            so, se = p.communicate(timeout=max(1, timeout - (time.time() - t0)))
        except subprocess.TimeoutExpired:
            p.kill()
            so, se = p.communicate()
            so += "\nTIMEOUT"
        lines = [l for l in so.splitlines() if l.startswith("RESULT ")]
        outs[r] = (p.returncode, json.loads(lines[-1][7:]) if lines else None, so[-500:] + se[-1500:])
    return outs, time.time() - t0


def test_root_cause_of_a_raising_rank_reaches_its_peer():
    outs, took = _launch(dict(mode="raise", bad_rank=1, fail_at=3), port=29810)
    rc1, res1, log1 = outs[1]
    assert res1 is not None and "synthetic failure" in res1["own_failure"], log1
    rc0, res0, log0 = outs[0]
    assert res0 is not None, log0
    # the survivor ends within seconds, knowing who failed and why (or, if it was already inside the collective, with that collective's error)
    assert took < 60
    if "remote_failure" in res0:
        assert res0["remote_failure"]["rank"] == 1 and "synthetic failure" in res0["remote_failure"]["reason"]
    else:
        assert "collective_error" in res0


def test_a_vanished_rank_is_detected_by_its_heartbeat():
    outs, took = _launch(dict(mode="exit", bad_rank=1, fail_at=3, stale_after_s=1.5, pg_timeout_s=8, abort_after_s=20), port=29820)
    assert outs[1][0] == 17
    rc0, res0, log0 = outs[0]
    assert took < 60
    # either the watchdog raised at the next check, or the collective timed out first, or the watchdog force-exited a stuck main thread (134)
    assert (res0 is not None and ("remote_failure" in res0 or "collective_error" in res0)) or rc0 == 134, log0
    if res0 is not None and "remote_failure" in res0:
        assert res0["remote_failure"]["rank"] == 1 and "heartbeat" in res0["remote_failure"]["reason"]


def test_watchdog_unit_with_in_process_store():
    from surogate_b200.parallel.watchdog import DictStore, RemoteRankFailed, Watchdog

    store = DictStore()
    aborted = []
    a = Watchdog(store, 0, 2, heartbeat_s=0.05, stale_after_s=0.4, abort_after_s=0.3, on_abort=aborted.append).start()
    b = Watchdog(store, 1, 2, heartbeat_s=0.05, stale_after_s=0.4, abort_after_s=None).start()
    time.sleep(0.3)
    a.check()
    b.check()
    try:
        with b.guard():
            raise KeyError("boom")
    except KeyError:
        pass
    time.sleep(0.3)
    with pytest.raises(RemoteRankFailed, match="KeyError"):
        a.check()
    a.stop()
    b.stop()
    # a silent peer: heartbeats stop, nobody calls check() -> the abort hook fires
    store2 = DictStore()
    c = Watchdog(store2, 0, 2, heartbeat_s=0.05, stale_after_s=0.3, abort_after_s=0.2, on_abort=aborted.append).start()
    d = Watchdog(store2, 1, 2, heartbeat_s=0.05, stale_after_s=10, abort_after_s=None).start()
    time.sleep(0.2)
    d._stop.set()  # rank 1 stops beating without saying goodbye
    time.sleep(1.2)
    assert aborted and "no heartbeat" in aborted[-1]
    c.stop()


def test_truncated_checkpoint_is_skipped_and_reported(tmp_path):
    from surogate_b200.io.checkpoint import find_latest_checkpoint, step_dir
    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    model = dict(architecture="Qwen3ForCausalLM", vocab_size=128, d_model=32, n_layers=1, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64,
                 tie_word_embeddings=True)
    tr = Trainer(TrainerConfig(model=model, batch_size=2, seq_len=16, optimizer="adamw", zero_level=0), device=torch.device("cpu"))
    tr.init_weights(0)
    tok = np.random.default_rng(0).integers(0, 128, (2, 17)).astype(np.int32)
    tr.step(tok[:, :-1], tok[:, 1:])
    tr.save_checkpoint(str(tmp_path), step=1)
    tr.step(tok[:, :-1], tok[:, 1:])
    tr.save_checkpoint(str(tmp_path), step=2)
    # a crash while writing step 3: the directory exists but checkpoint.json was never written
    os.makedirs(step_dir(str(tmp_path), 3))
    assert find_latest_checkpoint(str(tmp_path)) == 2
    # a torn weight shard of step 2: loading it must fail loudly, and step 1 still loads
    shard = [f for f in os.listdir(step_dir(str(tmp_path), 2)) if f.startswith("weights")][0]
    path = os.path.join(step_dir(str(tmp_path), 2), shard)
    with open(path, "r+b") as f:
        f.truncate(os.path.getsize(path) // 2)
    with pytest.raises(Exception):
        tr.load_checkpoint(str(tmp_path), 2)
    meta = tr.load_checkpoint(str(tmp_path), 1)
    assert meta["run"]["step"] == 1

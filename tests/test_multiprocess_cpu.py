"""Sharding math on CPU ranks (gloo): every ZeRO level at world size 2 reproduces the single-process run."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def run_worker(nproc, args, port=29611, timeout=240):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    if nproc == 1:
        cmd = [sys.executable, os.path.join(HERE, "mp_worker.py"), json.dumps(args)]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
               "--master-port", str(port), os.path.join(HERE, "mp_worker.py"), json.dumps(args)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


TINY = dict(architecture="Qwen3ForCausalLM", vocab_size=256, d_model=64, n_layers=2, num_query_heads=2, num_kv_heads=1, head_size=32, d_ff=128,
            tie_word_embeddings=True)


@pytest.fixture(scope="module")
def single():
    return run_worker(1, dict(device="cpu", model=TINY, global_batch=4, seq_len=32, steps=3))


@pytest.mark.parametrize("zero", [0, 1, 2, 3])
def test_zero_levels_match_single_process(single, zero):
    r = run_worker(2, dict(device="cpu", model=TINY, global_batch=4, seq_len=32, steps=3, zero=zero, keep_gathered=zero != 3), port=29611 + zero)
    assert r["world"] == 2
    for a, b in zip(r["losses"], single["losses"]):
        assert abs(a - b) < 2e-4 * abs(b), (r["losses"], single["losses"])
    for a, b in zip(r["norms"], single["norms"]):
        assert abs(a - b) < 1e-3 * abs(b), (r["norms"], single["norms"])


def test_grad_accumulation_with_sharded_gradients(single):
    r = run_worker(2, dict(device="cpu", model=TINY, global_batch=4, seq_len=32, steps=3, zero=2, grad_accum=2), port=29621)
    # same tokens per step, split into 2 micro-batches per rank of 1 row: rows are assigned differently, so compare loosely
    assert abs(r["losses"][0] - single["losses"][0]) < 5e-2


FOUR = dict(TINY, n_layers=4)


@pytest.mark.parametrize("tied,stage_layers,port", [(True, 0, 29641), (False, 1, 29642)])
def test_pipeline_stages_match_single_process(tmp_path, tied, stage_layers, port):
    """Layer ranges on two ranks, boundaries sent point to point, a diagonal wavefront of micro-batches: same losses and
    gradient norms as the unpartitioned run; with one layer per stage every rank interleaves two stages.  The tied
    embedding / LM-head weight is held by both end ranks and stays equal."""
    model = dict(FOUR, tie_word_embeddings=tied)
    one = run_worker(1, dict(device="cpu", model=model, global_batch=4, seq_len=32, steps=3, zero=0, grad_accum=2))
    out = os.path.join(tmp_path, "export")
    r = run_worker(2, dict(device="cpu", model=model, global_batch=4, seq_len=32, steps=3, pp=True, grad_accum=1, stage_layers=stage_layers, export_dir=out), port=port)
    assert r["world"] == 2 and len(r["stages"]) == (4 if stage_layers == 1 else 2)
    assert {s[2] for s in r["stages"]} == {0, 1}
    for a, b in zip(r["losses"], one["losses"]):
        assert abs(a - b) < 2e-4 * abs(b), (r["losses"], one["losses"])
    for a, b in zip(r["norms"], one["norms"]):
        assert abs(a - b) < 1e-3 * abs(b), (r["norms"], one["norms"])
    index = json.load(open(os.path.join(out, "model.safetensors.index.json")))
    names = set(index["weight_map"])
    assert {f"model.layers.{L}.mlp.down_proj.weight" for L in range(4)} <= names and "model.embed_tokens.weight" in names and "model.norm.weight" in names
    assert len(set(index["weight_map"].values())) == 2


def test_sft_loop_with_pipeline_stages_checkpoints_and_resumes(tmp_path):
    """`parallelism: dispatch_pp` through the SFT loop on two ranks: trains, evaluates, checkpoints per stage rank, exports a
    sharded HF directory and resumes from the per-stage checkpoints."""
    model = dict(architecture="Qwen3ForCausalLM", vocab_size=256, d_model=32, n_layers=2, num_query_heads=2, num_kv_heads=1, head_size=16, d_ff=64,
                 tie_word_embeddings=True)
    base = dict(model=json.dumps(model), synthetic_data=True, sequence_len=32, per_device_train_batch_size=2, gradient_accumulation_steps=1, max_steps=4,
                lora=False, optimizer="adamw", learning_rate=1e-2, save_steps=2, eval_steps=2, recipe="bf16", zero_level=0, from_scratch=True, parallelism="dispatch_pp",
                output_dir=str(tmp_path / "out"), report_to=[])

    def run(cfg, port):
        env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2", SUROGATE_NO_BANNER="1")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", str(port),
               os.path.join(HERE, "pp_sft_worker.py"), json.dumps(cfg)]
        p = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
        assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
        return json.loads([l for l in p.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])

    r = run(base, 29651)
    assert r["steps"] == 4 and all(l == l for l in r["losses"])
    out = tmp_path / "out"
    assert (out / "model.safetensors.index.json").exists() and (out / "stage_rank_000" / "step_00000002" / "checkpoint.json").exists()
    assert (out / "stage_rank_001" / "step_00000002" / "checkpoint.json").exists()
    r2 = run(dict(base, max_steps=6, save_steps=0, resume_from_checkpoint=True), 29652)
    assert r2["steps"] == 4  # resumed at step 2 of 6


@pytest.mark.parametrize("zero", [0, 2])
def test_lora_gradient_norm_on_two_ranks_equals_the_single_process_norm(zero):
    """The adapter gradient is all-reduced before the norm: it must be counted once, not once per rank (a norm sqrt(world) too
    large would over-clip and leave the 1-rank trajectory)."""
    lora = dict(rank=4, alpha=8, dropout=0.0, dtype="fp32", targets=["q_proj", "v_proj", "down_proj"], rslora=False, train_router=False)
    args = dict(device="cpu", model=TINY, global_batch=4, seq_len=32, steps=4, lora=lora)
    one = run_worker(1, dict(args, zero=0))
    two = run_worker(2, dict(args, zero=zero, keep_gathered=True), port=29661 + zero)
    assert two["world"] == 2
    for a, b in zip(two["norms"], one["norms"]):
        assert abs(a - b) < 2e-3 * abs(b), (two["norms"], one["norms"])
    for a, b in zip(two["losses"], one["losses"]):
        assert abs(a - b) < 2e-4 * abs(b), (two["losses"], one["losses"])


def test_checkpoint_write_failure_on_one_rank_is_abandoned_by_all_ranks(tmp_path):
    """Rank 1 cannot write its shard: both ranks raise the same error after the same collectives, no checkpoint.json appears, and
    the next training step still runs with the ranks in agreement."""
    from surogate_b200.io.checkpoint import find_latest_checkpoint

    r = run_worker(2, dict(device="cpu", model=TINY, global_batch=4, seq_len=32, steps=2, zero=2, checkpoint_dir=str(tmp_path), checkpoint_fail_rank=1), port=29671)
    assert r["checkpoint_all_ranks"] == ["CheckpointWriteError", "CheckpointWriteError"]
    assert find_latest_checkpoint(str(tmp_path)) is None
    assert r["loss_after"] == r["loss_after"] and r["loss_after"] > 0
    ok = run_worker(2, dict(device="cpu", model=TINY, global_batch=4, seq_len=32, steps=2, zero=2, checkpoint_dir=str(tmp_path)), port=29672)
    assert ok["checkpoint"] == "written" and find_latest_checkpoint(str(tmp_path)) == 2


MOE_TINY = dict(architecture="Qwen3MoeForCausalLM", vocab_size=256, d_model=64, n_layers=2, num_query_heads=2, num_kv_heads=1, head_size=32, moe_d_ff=32,
                num_experts=4, num_experts_per_tok=2, aux_loss_coef=0.0, tie_word_embeddings=False)   # (the load-balancing loss is a per-rank statistic)


@pytest.mark.parametrize("nproc,ep,zero,port", [(2, 2, 1, 29681), (2, 1, 1, 29682), (4, 2, 0, 29683), (4, 2, 2, 29684)])
def test_expert_parallel_mesh_matches_single_process(nproc, ep, zero, port):
    """Expert parallelism over the library all-to-all on CPU ranks: ep = world (one expert group), ep = 1 (pure data parallel) and the
    2 x 2 mesh (two replicas of a two-rank expert group: tokens dispatched inside a replica, expert gradients summed across replicas,
    every gradient counted once in the norm) all reproduce the single-process losses and gradient norms."""
    one = run_worker(1, dict(device="cpu", model=MOE_TINY, global_batch=4, seq_len=32, steps=3, zero=0))
    r = run_worker(nproc, dict(device="cpu", model=MOE_TINY, global_batch=4, seq_len=32, steps=3, zero=zero, ep=ep), port=port)
    assert r["world"] == nproc
    for a, b in zip(r["losses"], one["losses"]):
        assert abs(a - b) < 3e-4 * abs(b), (r["losses"], one["losses"])
    for a, b in zip(r["norms"], one["norms"]):
        assert abs(a - b) < 2e-3 * abs(b), (r["norms"], one["norms"])


def test_qlora_on_an_expert_parallel_model_keeps_frozen_experts_quantised():
    """QLoRA on a MoE model with EP=2 over CPU ranks: the frozen expert buckets are held by the expert offload manager (quantised, their
    master copies freed, rebuilt per layer when reached), training follows the run whose experts stay in full precision, and export
    still returns all experts."""
    lora = dict(rank=4, alpha=8, dropout=0.0, dtype="fp32", targets=["q_proj", "v_proj", "o_proj"], rslora=False, train_router=False)
    base = dict(device="cpu", model=MOE_TINY, global_batch=4, seq_len=32, steps=3, zero=0, ep=2, lora=lora, qlora="fp8_block")
    full = run_worker(2, dict(base, qlora_experts=False), port=29691)
    q = run_worker(2, dict(base, qlora_experts=True), port=29692)
    assert "expert_offload" not in full
    st = q["expert_offload"]
    assert st["expert_offload/layers"] == 2 and st["expert_offload/device_bytes_saved"] > 0 and q["expert_master_elems"] == 0
    assert q["exported_expert_shape"][0] == 4                      # all four experts come back from the two ranks
    for a, b in zip(q["losses"], full["losses"]):
        assert abs(a - b) < 2e-2 * abs(b), (q["losses"], full["losses"])


@pytest.mark.parametrize("nproc,port", [(2, 29693), (4, 29694)])
def test_least_loaded_spilling_keeps_the_math(nproc, port):
    """Per-step least-loaded balancing on the portable expert-parallel path: with a spill threshold of 1.0 every MoE layer of every step
    cuts the busiest experts' rows into chunks for helper ranks (weights shipped forward, weight gradients returned in backward);
    losses and gradient norms still equal the single-process run."""
    model = dict(MOE_TINY, num_experts=8)
    one = run_worker(1, dict(device="cpu", model=model, global_batch=4, seq_len=32, steps=3, zero=0))
    r = run_worker(nproc, dict(device="cpu", model=model, global_batch=4, seq_len=32, steps=3, zero=0, ep=nproc, ep_spill=1.0, ep_spill_min_rows=1), port=port)
    assert r["ep_spilled_layers"] >= 3, r["ep_spilled_layers"]
    for a, b in zip(r["losses"], one["losses"]):
        assert abs(a - b) < 3e-4 * abs(b), (r["losses"], one["losses"])
    for a, b in zip(r["norms"], one["norms"]):
        assert abs(a - b) < 2e-3 * abs(b), (r["norms"], one["norms"])


def test_biased_experts_under_expert_parallelism_with_and_without_spilling():
    """Experts with per-expert biases (GPT-OSS) on the portable expert-parallel path: the bias of a row is looked up in the RECEIVE
    plan's slot order, and on least-loaded steps the foreign slots' biases (and their gradients) travel like the weights."""
    model = dict(architecture="GptOssForCausalLM", vocab_size=256, d_model=64, n_layers=2, num_query_heads=2, num_kv_heads=1, head_size=32, d_ff=32,
                 num_experts=4, num_experts_per_tok=2, sliding_window=16, max_seq=128)
    one = run_worker(1, dict(device="cpu", model=model, global_batch=4, seq_len=32, steps=3, zero=0))
    plain = run_worker(2, dict(device="cpu", model=model, global_batch=4, seq_len=32, steps=3, zero=0, ep=2), port=29698)
    spill = run_worker(2, dict(device="cpu", model=model, global_batch=4, seq_len=32, steps=3, zero=0, ep=2, ep_spill=1.0, ep_spill_min_rows=1), port=29697)
    assert spill["ep_spilled_layers"] >= 3 and plain["ep_spilled_layers"] == 0
    for r in (plain, spill):
        for a, b in zip(r["losses"], one["losses"]):
            assert abs(a - b) < 3e-4 * abs(b), (r["losses"], one["losses"])
        for a, b in zip(r["norms"], one["norms"]):
            assert abs(a - b) < 2e-3 * abs(b), (r["norms"], one["norms"])

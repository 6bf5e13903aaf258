"""Two-GPU checks: NCCL collectives and the hand-written peer-memory collectives both reproduce the one-GPU run."""
import pytest

from test_multiprocess_cpu import run_worker

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

ARGS = dict(device="cuda", global_batch=4, seq_len=128, steps=4)


@pytest.fixture(scope="module")
def single():
    return run_worker(1, dict(ARGS))


@pytest.mark.parametrize("zero,collectives", [(1, "nccl"), (3, "nccl"), (1, "symm"), (2, "symm"), (3, "symm")])
def test_two_gpus_match_one_gpu(single, zero, collectives):
    r = run_worker(2, dict(ARGS, zero=zero, collectives=collectives, keep_gathered=zero != 3), port=29700 + zero + (10 if collectives == "symm" else 0))
    assert r["world"] == 2
    assert r["comm"] == ("SymmComm" if collectives == "symm" else "TorchComm")
    if collectives == "symm":
        assert r["fused_norm"], "gradient norm should come out of the fused reduce-scatter kernels"
    for a, b in zip(r["losses"], single["losses"]):
        assert abs(a - b) < 2e-2 * abs(b), (r["losses"], single["losses"])
    for a, b in zip(r["norms"], single["norms"]):
        assert abs(a - b) < 5e-2 * abs(b), (r["norms"], single["norms"])


def test_two_gpus_fp8_zero3_quantize_on_gather(single):
    """ZeRO-3 + FP8: the gather kernel writes E4M3 directly (same per-tensor scale as the separate quantiser would use),
    so the run matches the NCCL path that gathers bf16 and quantises afterwards."""
    import os

    os.environ["SUROGATE_FP8_SHARDS"] = "1"
    try:
        a = run_worker(2, dict(ARGS, zero=3, collectives="symm", recipe="fp8_hybrid", optimizer="adamw_8bit"), port=29731)
    finally:
        del os.environ["SUROGATE_FP8_SHARDS"]
    b = run_worker(2, dict(ARGS, zero=3, collectives="nccl", recipe="fp8_hybrid", optimizer="adamw_8bit"), port=29732)
    assert a["fp8_gather"] and not b["fp8_gather"]
    assert a["fp8_shards"], "each rank should publish an E4M3 copy of its own shard for the peers to pull"
    assert all(l == l for l in a["losses"])
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 5e-3 * abs(y), (a["losses"], b["losses"])
    # quantise on arrival (peers pull bf16) gives the same bytes: same scale, same rounding
    os.environ["SUROGATE_FP8_SHARDS"] = "0"
    try:
        c = run_worker(2, dict(ARGS, zero=3, collectives="symm", recipe="fp8_hybrid", optimizer="adamw_8bit"), port=29733)
    finally:
        del os.environ["SUROGATE_FP8_SHARDS"]
    assert c["fp8_gather"] and not c["fp8_shards"]
    for x, y in zip(a["losses"], c["losses"]):
        assert abs(x - y) < 1e-4 * abs(y), (a["losses"], c["losses"])


MOE = dict(architecture="Qwen3MoeForCausalLM", vocab_size=1024, d_model=256, n_layers=2, num_query_heads=2, num_kv_heads=1, head_size=128,
           moe_d_ff=128, num_experts=8, num_experts_per_tok=2, aux_loss_coef=1e-2, tie_word_embeddings=False)


def test_expert_parallel_matches_one_gpu():
    """EP=2: tokens are dispatched to the expert's owner by the peer-memory kernels; the run reproduces the 1-GPU run."""
    one = run_worker(1, dict(ARGS, model=MOE))
    two = run_worker(2, dict(ARGS, model=MOE, ep=2, zero=1, collectives="symm"), port=29741)
    for a, b in zip(two["losses"], one["losses"]):
        assert abs(a - b) < 2e-2 * abs(b), (two["losses"], one["losses"])
    for a, b in zip(two["norms"], one["norms"]):
        assert abs(a - b) < 6e-2 * abs(b), (two["norms"], one["norms"])


def test_expert_parallel_with_fp8_experts_trains_like_one_gpu():
    """EP=2 under the FP8 recipe: the dispatched rows are quantised up to the device-side row count and run through the grouped FP8
    GEMMs on the expert's owner; losses follow the 1-GPU FP8 run."""
    import os

    one = run_worker(1, dict(ARGS, model=MOE, recipe="fp8_hybrid"))
    os.environ["SUROGATE_EP_FP8_DISPATCH"] = "0"
    try:
        two = run_worker(2, dict(ARGS, model=MOE, recipe="fp8_hybrid", ep=2, zero=1, collectives="symm"), port=29743)
    finally:
        del os.environ["SUROGATE_EP_FP8_DISPATCH"]
    for a, b in zip(two["losses"], one["losses"]):
        assert abs(a - b) < 4e-2 * abs(b), (two["losses"], one["losses"])
    # the default: rows quantised by the sender (E4M3 over NVLink with the expert group's shared delayed scale, from the second step on)
    q = run_worker(2, dict(ARGS, model=MOE, recipe="fp8_hybrid", ep=2, zero=1, collectives="symm"), port=29744)
    assert q["fp8_dispatches"] > 0 and two["fp8_dispatches"] == 0
    assert q["losses"][0] == two["losses"][0]            # the first step has no scale yet: same path
    for a, b in zip(q["losses"], two["losses"]):
        assert abs(a - b) < 2e-2 * abs(b), (q["losses"], two["losses"])


LORA = dict(rank=8, alpha=16, dropout=0.0, dtype="fp32", targets=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"],
            rslora=False, train_router=False)


@pytest.mark.parametrize("collectives", ["nccl", "symm"])
def test_two_gpus_lora_zero3_host_resident_base(collectives):
    """LoRA over a frozen base whose shards live in pinned host memory: H2D into a peer-visible slot + peer-memory gather
    (or H2D + NCCL) reproduces the run with device-resident weights."""
    ref = run_worker(2, dict(ARGS, zero=3, collectives=collectives, lora=LORA, keep_gathered=False), port=29751)
    off = run_worker(2, dict(ARGS, zero=3, collectives=collectives, lora=LORA, keep_gathered=False, offload_master=True, offload_optimizer=True),
                     port=29752)
    assert off["h2d_weight_bytes"] > 0
    if collectives == "symm":
        assert off["stage_slots"] == 2
    for a, b in zip(off["losses"], ref["losses"]):
        assert abs(a - b) < 1e-3 * abs(b), (off["losses"], ref["losses"])


def test_two_gpus_full_finetune_offloaded_state():
    ref = run_worker(2, dict(ARGS, zero=3, collectives="symm", optimizer="adamw_8bit", keep_gathered=False), port=29753)
    off = run_worker(2, dict(ARGS, zero=3, collectives="symm", optimizer="adamw_8bit", keep_gathered=False, offload_master=True, offload_optimizer=True),
                     port=29754)
    for a, b in zip(off["losses"], ref["losses"]):
        assert abs(a - b) < 5e-3 * abs(b), (off["losses"], ref["losses"])


def test_expert_parallel_overflow_drops_tokens_instead_of_overrunning():
    """A receive buffer far too small for the routed rows: the overflow is dropped and counted, nothing is written or read
    outside the buffer, and training continues with finite numbers."""
    r = run_worker(2, dict(ARGS, global_batch=8, seq_len=256, model=MOE, ep=2, zero=1, collectives="symm", ep_capacity_factor=0.05), port=29761)
    assert r["ep_dropped"] > 0
    assert all(l == l and abs(l) < 50 for l in r["losses"]), r["losses"]


def test_expert_replacement_keeps_the_trajectory():
    """Least-loaded placement: experts (weights + optimizer moments) move between ranks every 2 steps with a threshold that
    always triggers; the run must still reproduce the 1-GPU trajectory, because only WHERE an expert lives changes."""
    args = dict(ARGS, model=MOE, steps=6, optimizer="adamw_8bit")
    one = run_worker(1, dict(args))
    two = run_worker(2, dict(args, ep=2, zero=1, collectives="symm", ep_refresh=2, ep_threshold=1.0), port=29771)
    assert two["ep_moves"] > 0
    for a, b in zip(two["losses"], one["losses"]):
        assert abs(a - b) < 2e-2 * abs(b), (two["losses"], one["losses"])


@pytest.mark.parametrize("stage_layers", [0, 1])
def test_pipeline_stages_on_two_gpus_match_one_gpu(stage_layers):
    """Layer ranges per GPU with boundaries sent peer to peer (NCCL send / recv over NVLink): the trajectory of the one-GPU run
    with the same micro-batches.  ``stage_layers=1`` interleaves two stages per GPU, so both directions of the link are in use
    in the same tick."""
    model = dict(architecture="Qwen3ForCausalLM", vocab_size=1024, d_model=256, n_layers=4, num_query_heads=2, num_kv_heads=1, head_size=128, d_ff=512,
                 tie_word_embeddings=True)
    one = run_worker(1, dict(ARGS, model=model, zero=0, grad_accum=2))
    r = run_worker(2, dict(ARGS, model=model, pp=True, grad_accum=1, stage_layers=stage_layers), port=29781 + stage_layers)
    assert r["world"] == 2 and len(r["stages"]) == (4 if stage_layers else 2)
    for a, b in zip(r["losses"], one["losses"]):
        assert abs(a - b) < 2e-2 * abs(b), (r["losses"], one["losses"])
    for a, b in zip(r["norms"], one["norms"]):
        assert abs(a - b) < 5e-2 * abs(b), (r["norms"], one["norms"])


@pytest.mark.parametrize("collectives", ["nccl", "symm"])
def test_two_gpus_graph_replay_with_deferred_reductions(single, collectives):
    """Forward + backward replayed from CUDA graphs on each rank, gradient reduce-scatter issued after the replay."""
    r = run_worker(2, dict(ARGS, zero=1, collectives=collectives, graphs=True, steps=6), port=29785 + (1 if collectives == "symm" else 0))
    one = run_worker(1, dict(ARGS, steps=6))
    assert r["graph_replays"] == 4, r["graph_replays"]
    for a, b in zip(r["losses"], one["losses"]):
        assert abs(a - b) < 2e-2 * abs(b), (r["losses"], one["losses"])

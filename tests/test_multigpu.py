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


def test_two_gpus_fp8_zero3_symm(single):
    r = run_worker(2, dict(ARGS, zero=3, collectives="symm", recipe="fp8_hybrid", optimizer="adamw_8bit"), port=29731)
    assert all(l == l for l in r["losses"]) and r["losses"][-1] < r["losses"][0] + 0.5

"""Device-timed bandwidth of the peer-memory collectives against NCCL, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m surogate_b200.utils.collective_bench [--mib 64 256]

For each bucket size: the fused reduce-scatter (+ scale + sum of squares) and the all-gather (bf16, and with FP8 quantise-on-gather)
of ``csrc/comm_kernels.cu`` and NCCL's reduce_scatter_tensor / all_gather_into_tensor on the same buffers.  Every figure is
the mean of ``--iters`` launches after warm-up, timed with CUDA events on the launching stream, max over ranks.  Reported per
rank: bytes that must cross NVLink, (N-1)/N of the bucket, divided by the time, and that as a fraction of the measured peer-copy
bandwidth of this pool (770 GB/s per direction) — the roofline of a collective whose arithmetic is negligible.  The buckets
alternate between two arena regions larger than the L2, so no launch finds its input cached.
"""
from __future__ import annotations

import argparse
import json
from typing import Callable, Dict, List

import torch

NVLINK_GBS = 770.0  # measured peer copy, per direction per GPU


def _time(fn: Callable[[int], None], iters: int, warmup: int, comm) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    comm.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    ms = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
    return float(ms)


def _expert_parallel_cases(a, comm, dev) -> List[Dict]:
    """Dispatch (routing permutation + peer stores) and combine (peer loads + weighted sum) of one MoE layer with uniform random routing:
    every rank sends ``tokens x top_k`` rows of ``hidden`` bf16 values, (world - 1) / world of them over NVLink."""
    from ..parallel.ep import SLOT_EP, ExpertParallel

    world = comm.world
    N, K, E, C = a.ep_tokens, a.ep_topk, a.ep_experts, a.ep_hidden
    if E % world:
        return []
    ep = ExpertParallel(comm, world, dev, capacity_factor=float(min(world, 3)))
    b = ep._ensure(N, K, C, E)
    El, cap = b["El"], b["cap"]
    g = torch.Generator(device="cuda").manual_seed(comm.rank)
    x = torch.randn(N, C, device=dev, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(E, device=dev, generator=g)[:K] for _ in range(N)]).to(torch.int32).contiguous()
    counts = torch.bincount(idx.reshape(-1).long(), minlength=E).to(torch.int32)
    w = torch.rand(N, K, device=dev, generator=g)
    offsets = torch.zeros(2 * El + 2, dtype=torch.int32, device=dev)
    dst_base = torch.empty(E, dtype=torch.int32, device=dev)
    cursors = torch.empty(E, dtype=torch.int32, device=dev)
    row_map = torch.empty(N * K, dtype=torch.int32, device=dev)
    pb = b["arena"].peer_bases
    ext = comm.ext

    def plan(i):
        ep.epoch += 1
        ext.ep_plan(pb, b["counts_off"], comm.ctrl.peer_bases, counts, offsets, dst_base, cursors, comm.rank, ep.epoch & 0x7FFFFFFF, SLOT_EP, cap, comm.err,
                    comm.wait_budget_s)

    def dispatch(i):
        plan(i)
        pos = ext.ep_row_positions(idx.reshape(-1), E)
        ext.ep_dispatch(x, idx, None, dst_base, pos, row_map, pb, b["recv_x_off"], K, El, cap, False)
        comm.fence()

    def combine(i):
        ext.ep_combine(pb, b["out_y_off"], w, row_map, N, C, K, cap, False)
        comm.fence()

    dispatch(0)
    ext.copy_rows_upto(b["recv_x"], b["out_y"], offsets[El:El + 1])   # something to pull back
    comm.fence()
    cross = (world - 1) / world * N * K * C * 2
    out = []
    for name, fn in (("ep dispatch (plan + permutation + peer stores + barrier)", dispatch), ("ep combine (peer loads + weighted sum + barrier)", combine)):
        ms = _time(fn, a.iters, a.warmup, comm)
        gbs = cross / ms / 1e6
        out.append({"case": name, "tokens_per_rank": N, "top_k": K, "hidden": C, "ranks": world, "ms": round(ms, 4), "nvlink_gb_s_per_rank": round(gbs, 1),
                    "fraction_of_measured_peer_copy": round(gbs / NVLINK_GBS, 3)})
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, nargs="+", default=[64, 256], help="bucket sizes (bf16 bytes, whole bucket)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--multimem", action="store_true", help="also time the NVLS (multimem) reduce-scatter; leave off in runs where a rank may leave early")
    ap.add_argument("--ep-tokens", type=int, default=4096, help="tokens per rank for the expert-parallel dispatch / combine case (0 = skip)")
    ap.add_argument("--ep-hidden", type=int, default=2048)
    ap.add_argument("--ep-experts", type=int, default=128)
    ap.add_argument("--ep-topk", type=int, default=8)
    a = ap.parse_args(argv)

    from ..parallel import symm
    from ..parallel.dist import TorchComm, init_distributed

    info = init_distributed()
    dev = torch.device("cuda", info.local_rank)
    torch.cuda.set_device(dev)
    base = TorchComm()
    comm = symm.try_create(base, dev, required=True)
    world, rank = comm.world, comm.rank
    rows: List[Dict] = []
    biggest = max(a.mib) << 20
    arena = comm.create_arena(2 * biggest + 2 * (biggest // world) + (1 << 20))
    for mib in a.mib:
        nbytes = mib << 20
        n = nbytes // 2
        n -= n % (world * 1024)
        sh = n // world
        fulls = [arena.take(n, torch.bfloat16) for _ in range(2)]
        shards_sym = [arena.take(sh, torch.bfloat16) for _ in range(2)]
        for f in fulls:
            f.normal_()
        for s in shards_sym:
            s.normal_()
        shard = torch.empty(sh, dtype=torch.bfloat16, device=dev)
        out_full = torch.empty(n, dtype=torch.bfloat16, device=dev)
        out_fp8 = torch.empty(n, dtype=torch.uint8, device=dev)
        sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        scale = torch.ones(1, dtype=torch.float32, device=dev)
        cross = (world - 1) / world * n * 2  # bytes per rank over NVLink, both collectives (bf16)
        def rs_multimem(i):
            comm.use_multimem = True
            try:
                comm.reduce_scatter(fulls[i & 1], shard, sumsq_out=sumsq)
            finally:
                comm.use_multimem = False

        cases = {
            "reduce_scatter fused (+scale +sumsq)": (lambda i: comm.reduce_scatter(fulls[i & 1], shard, sumsq_out=sumsq), cross),
            "reduce_scatter NCCL": (lambda i: base.reduce_scatter(fulls[i & 1], shard), cross),
            "all_gather fused bf16": (lambda i: comm.all_gather(shards_sym[i & 1], out_full), cross),
            "all_gather fused + FP8 quantise": (lambda i: comm.all_gather(shards_sym[i & 1], None, out_fp8=out_fp8, scale=scale), cross),
            "all_gather NCCL": (lambda i: base.all_gather(shards_sym[i & 1], out_full), cross),
        }
        if a.multimem and arena.mc_base:   # in-switch reduction (NVLS): every rank reads the reduced value of its shard through the multicast address
            cases["reduce_scatter multimem (+scale +sumsq)"] = (rs_multimem, cross)
        for name, (fn, nb) in cases.items():
            ms = _time(fn, a.iters, a.warmup, comm)
            gbs = nb / ms / 1e6
            rows.append({"case": name, "bucket_mib": mib, "ranks": world, "ms": round(ms, 4), "nvlink_gb_s_per_rank": round(gbs, 1),
                         "fraction_of_measured_peer_copy": round(gbs / NVLINK_GBS, 3)})
        arena.cursor = 0  # the next size reuses the arena
    if a.ep_tokens > 0:
        rows.extend(_expert_parallel_cases(a, comm, dev))
    from ..ops import check_device_errors

    check_device_errors()
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

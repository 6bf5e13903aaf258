"""Expert re-placement moves (weights + optimizer state of experts changing owner) as one all-to-all over four CPU ranks."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from types import SimpleNamespace

    from surogate_b200.parallel.ep import ExpertParallel

    E, El, per = 8, 2, 256                      # 8 experts, 2 slots per rank, 256 weights per expert and slot
    slots = [SimpleNamespace(offset=0, numel=El * per), SimpleNamespace(offset=El * per, numel=El * per)]    # two parameters (gate_up, down)
    cur = list(range(E))                         # expert e sits in global slot e
    new = [2, 1, 4, 3, 6, 5, 0, 7]               # 0 -> rank 1, 2 -> rank 2, 4 -> rank 3, 6 -> rank 0: a cycle through all four ranks
    new[1], new[0] = new[0], new[1]              # and a swap inside rank 0's pair: expert 0 -> slot 1?, keep it a permutation
    assert sorted(new) == list(range(E))

    def content(e, p, kind):                     # what expert e's part p of tensor kind holds: recognisable anywhere
        n = per if kind != "scale" else per // 32
        return torch.full((n,), float(e * 10 + p + {"master": 0.0, "m": 0.25, "scale": 0.5}[kind]))

    def build(dtype, kind):
        n = (2 * El * per) if kind != "scale" else (2 * El * per) // 32
        t = torch.zeros(n, dtype=dtype)
        for p, sl in enumerate(slots):
            for s_local in range(El):
                e = cur.index(rank * El + s_local)
                seg = per if kind != "scale" else per // 32
                off = (sl.offset + s_local * per) // (1 if kind != "scale" else 32)
                t[off:off + seg] = content(e, p, kind).to(dtype)
        return t

    master, m8, scale = build(torch.float32, "master"), build(torch.float32, "m").to(torch.bfloat16), build(torch.float16, "scale")
    bucket = SimpleNamespace(name="layer0.experts", master=master, work=master, slots=slots)
    store = SimpleNamespace(buckets={"layer0.experts": bucket})
    optimizer = SimpleNamespace(state={"layer0.experts": {"m": m8, "m.scales": scale}})
    ep = object.__new__(ExpertParallel)
    ep.ep, ep.rank = world, rank
    ep.comm = SimpleNamespace(base=SimpleNamespace(group=None))
    ep._move_experts(store, optimizer, 0, cur, new, El, dist)
    ok = True
    for p, sl in enumerate(slots):
        for s_local in range(El):
            e = new.index(rank * El + s_local)   # who lives here now
            a = sl.offset + s_local * per
            ok &= bool(torch.equal(master[a:a + per], content(e, p, "master")))
            ok &= bool(torch.equal(m8[a:a + per].float(), content(e, p, "m").to(torch.bfloat16).float()))
            ok &= bool(torch.equal(scale[a // 32:(a + per) // 32].float(), content(e, p, "scale").to(torch.float16).float()))
    # a layer in which nothing moves for this rank's pairs still completes when every rank enters the call
    ep._move_experts(store, optimizer, 0, new, new, El, dist)
    with open(os.path.join(out_dir, f"r{rank}"), "w") as f:
        f.write("ok" if ok else "bad")
    dist.barrier()
    dist.destroy_process_group()


def test_moves_over_four_ranks_deliver_every_experts_state(tmp_path):
    world = 4
    mp.spawn(_worker, args=(world, 29791, str(tmp_path)), nprocs=world, join=True)
    assert [open(tmp_path / f"r{r}").read() for r in range(world)] == ["ok"] * world

"""Expert parallelism over symmetric memory: token dispatch / combine done by this framework's own kernels.

Mesh: ``world = dp x ep`` with ``ep_rank = rank % ep`` (parallel/mesh.py).  ``comm`` is the symmetric-memory communicator of ONE
expert group: the whole world when ``dp = 1``, otherwise the sub-group of ``ep`` consecutive ranks (every rank owns ``E / ep`` experts
of every MoE layer; all non-expert parameters are data-parallel over the world, expert gradients over the replicas).  Per MoE layer, forward:

1. ``ep_plan``     counts exchange (P2P stores + in-kernel flag barrier) -> padded receive layout and per-expert write cursors,
2. ``ep_dispatch`` each token's activation row is stored straight into the owning rank's receive buffer (routing
                   permutation and all-to-all are the same pass),
3. grouped tcgen05 GEMMs over the received rows (device-side offsets, no host read of any count),
4. ``ep_combine``  every token pulls its K expert outputs from the owners and forms the weighted sum.

Backward runs the mirror image (push ``w * dy`` to the owners, grouped dgrad/wgrad there, pull ``d_x`` back).  Four
symmetric buffers (receive / output for activations and for gradients) are allocated once and reused by every layer;
the in-kernel barrier of step 1 (and an explicit one in backward) also guarantees that every rank is done with the
previous layer's buffers before they are overwritten.  The receive capacity is ``capacity_factor x tokens x K`` rows
(+ padding); token copies beyond it are dropped (they contribute zero to the combine) and counted per layer.

Least-loaded balancing: per-expert global token counts of every layer are kept from the last step
(``last_global_counts``) and summarised by ``imbalance()``; the LPT planner in :mod:`surogate_b200.parallel.lpt`
turns them into an expert->rank placement that the next re-shard applies.

Parity: csrc/src/runtime/ep/ep_strategy.cpp:1347-1980 (dispatch_forward / combine), lpt_planner.h:56-80,
csrc/src/utilities/comm.cpp:515-646 (EP groups, variable-split all-to-all).
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

SLOT_EP = 24  # signal-pad channel used by the in-kernel barrier of ep_plan (compute stream)


class EpPlan:
    def __init__(self, offsets, row_map, capacity, num_tokens, top_k, x_shape, topk_idx):
        self.offsets, self.row_map, self.capacity = offsets, row_map, capacity
        self.num_tokens, self.top_k, self.x_shape, self.topk_idx = num_tokens, top_k, x_shape, topk_idx
        self.kept_rows = None
        self.local = None
        self.ep = True


class PrePlan:
    """Output of moe_permute under EP: nothing is moved yet, the dispatch kernel permutes while it sends."""

    def __init__(self, topk_idx, counts, num_tokens, top_k, num_experts, x_shape):
        self.topk_idx, self.counts, self.num_tokens, self.top_k, self.num_experts, self.x_shape = topk_idx, counts, num_tokens, top_k, num_experts, x_shape
        self.local = None
        self.ep_plan = None


def decide_placement(placed_counts, cur, ep: int, threshold: float = 1.3, tolerance: float = 0.05, min_gain: float = 0.25, max_moved_fraction: float = 0.5):
    """New placement of one layer's experts, or the current one when moving is not worth it.

    ``placed_counts[i]`` is the number of routed rows of the expert held at placed index i (rank * El + slot); ``cur[e]`` is the
    placed index of global expert e.  Nothing moves when the busiest rank is within ``threshold`` of the mean, when the planner's
    proposal removes less than the fraction ``min_gain`` of the excess over a perfect balance, or when it would move more than ``max_moved_fraction`` of the
    experts at once (a sign that the counts are noise, not a stable skew).  Returns (placement, number of experts moved)."""
    from ..ops import host

    E = len(cur)
    El = E // ep
    counts = [placed_counts[cur[e]] for e in range(E)]  # per global expert

    def imbalance(place):
        per_rank = [0] * ep
        for e, c in enumerate(counts):
            per_rank[place[e] // El] += c
        return max(per_rank) / max(1.0, sum(per_rank) / ep)

    before = imbalance(cur)
    if before <= threshold:
        return list(cur), 0
    new, moved = host().balanced_placement(counts, ep, list(cur), tolerance)
    new = list(new)
    if moved == 0 or moved > max(1, int(max_moved_fraction * E)) or before - imbalance(new) < min_gain * (before - 1.0):
        return list(cur), 0
    return new, int(moved)


class PlacementBackoff:
    """Keeps re-placement from chasing noise.  The window after a move shows what the move was worth: if the layer's rank
    imbalance did not drop by a tenth, its counts are noise rather than a stable skew, and the layer sits out 1, 2, 4, then 8
    refreshes (doubling each time a move fails again); a move that helped resets the pause."""

    def __init__(self, needed_drop: float = 0.1, max_pause: int = 8):
        self.needed_drop, self.max_pause = needed_drop, max_pause
        self.state: Dict[int, list] = {}  # layer -> [imbalance before the last move (None once judged), refreshes left to sit out, last pause length]

    def sits_out(self, layer: int, imbalance_now: float) -> bool:
        st = self.state.get(layer)
        if st is None:
            return False
        if st[0] is not None:  # first refresh after a move: judge it
            helped = imbalance_now <= (1.0 - self.needed_drop) * st[0]
            st[2] = 0 if helped else min(self.max_pause, max(1, 2 * st[2]))
            st[0], st[1] = None, st[2]
        if st[1] > 0:
            st[1] -= 1
            return True
        return False

    def moved(self, layer: int, imbalance_before: float) -> None:
        st = self.state.get(layer)
        self.state[layer] = [imbalance_before, 0, st[2] if st is not None else 0]


class ExpertParallel:
    def __init__(self, comm, ep_size: int, device, capacity_factor: float = 1.5):
        if not hasattr(comm, "create_arena"):
            raise RuntimeError("expert parallelism needs the symmetric-memory communicator (collectives: symm)")
        if ep_size != comm.world:
            raise ValueError(f"the expert group's communicator has {comm.world} ranks but ep_size is {ep_size} "
                             "(with ep_size < world the trainer passes the sub-group communicator of parallel/mesh.py)")
        self.comm, self.ep, self.rank, self.device = comm, ep_size, comm.rank, device
        self.capacity_factor = capacity_factor
        self.ext = comm.ext
        self.err = comm.err
        self.bufs: Optional[Dict[str, Any]] = None
        self.epoch = 0
        self.last_global_counts: Dict[int, torch.Tensor] = {}
        self.count_window: Dict[int, torch.Tensor] = {}
        self.last_overflow: Dict[int, torch.Tensor] = {}  # rows per layer that exceeded this rank's receive capacity (dropped)
        # Least-loaded placement: placement[layer][e] = rank * El + slot that currently holds global expert e (identity at start).
        self.placement: Dict[int, torch.Tensor] = {}
        self.placement_host: Dict[int, list] = {}
        self.moves_done = 0

    # ------------------------------------------------------------------ buffers
    def _ensure(self, tokens: int, K: int, C: int, E: int):
        if self.bufs is not None:
            return self.bufs
        El = E // self.ep
        cap = int(self.capacity_factor * tokens * K) + El * 128
        cap = (cap + 127) // 128 * 128
        row_bytes = C * 2
        sizes = {"counts": self.ep * E * 4, "recv_x": cap * row_bytes, "out_y": cap * row_bytes, "recv_dy": cap * row_bytes, "out_dx": cap * row_bytes}
        total = sum((v + 255) // 256 * 256 + 256 for v in sizes.values())
        arena = self.comm._alloc_symmetric(total)
        arena.tensor.zero_()
        b: Dict[str, Any] = {"arena": arena, "cap": cap, "C": C, "E": E, "El": El}
        for k, n in sizes.items():
            t = arena.take(n, torch.uint8)
            b[k] = t.view(torch.int32) if k == "counts" else t.view(torch.bfloat16).view(cap, C)
            b[k + "_off"] = arena.offset_of(t)
        torch.cuda.synchronize(self.device)
        self.comm.base.barrier()
        self.bufs = b
        return b

    def _barrier(self):
        self.comm.fence()

    # ------------------------------------------------------------------ forward
    def dispatch(self, ctx, x2: torch.Tensor, pre: PrePlan):
        N, K, E = pre.num_tokens, pre.top_k, pre.num_experts
        C = x2.shape[-1]
        b = self._ensure(N, K, C, E)
        cap, El = b["cap"], b["El"]
        dev = x2.device
        offsets = torch.zeros(2 * El + 2, dtype=torch.int32, device=dev)  # El+1 padded row starts, overflow count, El real row counts
        dst_base = torch.empty(E, dtype=torch.int32, device=dev)
        cursors = torch.empty(E, dtype=torch.int32, device=dev)
        row_map = torch.empty(N * K, dtype=torch.int32, device=dev)
        self.epoch += 1
        pb = b["arena"].peer_bases
        self.ext.ep_plan(pb, b["counts_off"], self.comm.ctrl.peer_bases, pre.counts, offsets, dst_base, cursors, self.rank, self.epoch & 0x7FFFFFFF,
                         SLOT_EP, cap, self.err, self.comm.wait_budget_s)
        rec = getattr(ctx, "recipe", None)
        fp8 = rec.dispatch_fp8(ctx, x2) if (rec is not None and hasattr(rec, "dispatch_fp8")) else None
        # FP8 rows are one byte per element: the same receive buffer seen as [cap, C] bytes = [cap, C / 2] 16-bit units, so the
        # row-wise helpers (pad clearing, copy of the rows in use) work on it unchanged
        recv = b["recv_x"] if fp8 is None else b["recv_x"].view(-1).view(torch.uint8)[:cap * C].view(torch.bfloat16).view(cap, C // 2)
        # pad rows feed the wgrad contraction and must be zero; only they are touched, so peers may already be storing real rows
        self.ext.ep_zero_pad_rows(recv, offsets, El, cap)
        # rows are taken in token order (a stable counting sort per expert), not claimed with atomics: same layout in every run
        row_pos = self.ext.ep_row_positions(pre.topk_idx.reshape(-1).contiguous(), E)
        if fp8 is None:
            self.ext.ep_dispatch(x2.contiguous(), pre.topk_idx, None, dst_base, row_pos, row_map, pb, b["recv_x_off"], K, El, cap, False)
        else:
            self.ext.ep_dispatch(x2.contiguous(), pre.topk_idx, None, dst_base, row_pos, row_map, pb, b["recv_x_off"], K, El, cap, False, fp8[0], fp8[2])
        self._barrier()  # every rank's rows have landed
        xp = torch.empty_like(recv)         # rows beyond the used range stay uninitialised: nothing downstream reads them into a result
        used = offsets[El:El + 1]           # padded rows in use this step (device side): element-wise kernels downstream stop there
        self.ext.copy_rows_upto(recv, xp, used)
        if fp8 is not None:
            xp = xp.view(torch.uint8).view(cap, C).view(torch.float8_e4m3fn)
            xp._sg_inv = fp8[1]
            self.fp8_dispatches = getattr(self, "fp8_dispatches", 0) + 1
        xp._sg_rows = used
        if ctx.layer is not None and ctx.phase == "fwd":
            gc = b["counts"].view(self.ep, E).sum(0)
            self.last_global_counts[ctx.layer] = gc
            acc = self.count_window.get(ctx.layer)  # counts summed since the last placement refresh: what re-placement decides on
            if acc is None:
                self.count_window[ctx.layer] = gc.to(torch.int64).clone()
            else:
                acc.add_(gc)
            self.last_overflow[ctx.layer] = offsets[El + 1:El + 2]
        plan = EpPlan(offsets[:El + 1], row_map, cap, N, K, pre.x_shape, pre.topk_idx)
        plan.layout = offsets
        pre.ep_plan = plan
        return xp, plan

    def publish_outputs(self, ctx, h: torch.Tensor, plan: EpPlan, backward: bool = False):
        """Expert outputs (or d_x of the experts in backward) become visible to the token owners."""
        b = self.bufs
        buf = b["out_dx"] if backward else b["out_y"]
        self.ext.copy_rows_upto(h.contiguous(), buf, plan.layout[b["El"]:b["El"] + 1])
        self._barrier()
        return buf

    def combine(self, ctx, buf: torch.Tensor, weights: Optional[torch.Tensor], plan: EpPlan, backward: bool = False):
        b = self.bufs
        off = b["out_dx_off"] if backward else b["out_y_off"]
        w = weights.reshape(-1, plan.top_k).contiguous() if weights is not None else None
        y, rows = self.ext.ep_combine(b["arena"].peer_bases, off, w, plan.row_map, plan.num_tokens, b["C"], plan.top_k, plan.capacity,
                                      (not backward) and ctx.training)
        if rows is not None and rows.numel():
            plan.kept_rows = rows
        return y.reshape(plan.x_shape)

    # ------------------------------------------------------------------ backward
    def combine_backward(self, ctx, dy: torch.Tensor, weights: torch.Tensor, plan: EpPlan):
        """d_yp rows (w * dy) are pushed to the experts' owners; d_weights come from the rows kept in forward."""
        b = self.bufs
        K = plan.top_k
        dy2 = dy.reshape(plan.num_tokens, -1).contiguous()
        w = weights.reshape(-1, K).contiguous()
        d_w = self.ext.ep_weight_grad(plan.kept_rows, dy2, K)
        self._barrier()  # peers are done with the previous contents of their gradient buffers
        self.ext.ep_zero_pad_rows(b["recv_dy"], plan.layout, b["El"], plan.capacity)
        self.ext.ep_dispatch(dy2, None, w, None, None, plan.row_map, b["arena"].peer_bases, b["recv_dy_off"], K, b["El"], plan.capacity, True)
        self._barrier()
        dyp = torch.empty_like(b["recv_dy"])
        used = plan.layout[b["El"]:b["El"] + 1]
        self.ext.copy_rows_upto(b["recv_dy"], dyp, used)
        dyp._sg_rows = used
        return dyp, d_w.reshape(weights.shape)

    # ------------------------------------------------------------------ least-loaded expert placement
    def place(self, layer, topk_idx: torch.Tensor, counts: torch.Tensor):
        """Router output (global expert ids, per-expert counts) -> ids / counts in placed order, which is what the dispatch
        kernels understand (owner = id // El, local slot = id % El)."""
        p = self.placement.get(layer)
        if p is None:
            return topk_idx, counts
        placed = p[topk_idx.long()]
        c = torch.zeros_like(counts).scatter_(0, p.long(), counts)
        return placed.contiguous(), c

    def rebalance(self, store, optimizer, threshold: float = 1.3, tolerance: float = 0.05) -> Dict[str, Any]:
        """Re-place experts so that every rank sees about the same number of routed rows (from the counts summed over the steps
        since the last refresh, which smooths the step-to-step noise of the router).

        Ownership itself moves: the expert's master weights, work weights and optimizer moments travel to the new owner
        (point-to-point over NCCL, once per refresh), so later steps need no per-step weight shipping or gradient return.
        Layers whose rank imbalance is below ``threshold`` are left alone.  Collective: every rank must call it."""
        import torch.distributed as dist

        from ..ops import host

        if not self.count_window:
            return {"layers": 0, "moved": 0}
        if getattr(store, "expert_offload", None) is not None:
            # frozen experts held quantised (possibly in host memory): their placement is fixed, moving them would mean re-quantising
            for w in self.count_window.values():
                w.zero_()
            return {"layers": 0, "moved": 0, "skipped": "quantised experts"}
        layers = sorted(self.count_window)
        stacked = torch.stack([self.count_window[L] for L in layers])
        replica_comm = getattr(self, "replica_comm", None)
        if replica_comm is not None and replica_comm.world > 1:
            replica_comm.all_reduce(stacked, "sum")   # every replica of the expert group must take the same decision: decide on the global counts
        counts_all = stacked.cpu()  # the one host sync of a refresh
        E = counts_all.shape[1]
        El = E // self.ep
        changed, moved_total = 0, 0
        backoff = self.__dict__.setdefault("_backoff", PlacementBackoff())
        for li, L in enumerate(layers):
            cur = self.placement_host.get(L) or list(range(E))
            counts = counts_all[li].tolist()
            self.count_window[L].zero_()  # a new window starts (and counts are kept in placed order, which may change now)
            per_rank = [sum(counts[r * El:(r + 1) * El]) for r in range(self.ep)]
            now = max(per_rank) / max(1.0, sum(per_rank) / self.ep)
            if backoff.sits_out(L, now):
                continue
            new, moved = decide_placement(counts, cur, self.ep, threshold, tolerance)
            if moved == 0:
                continue
            backoff.moved(L, now)
            self._move_experts(store, optimizer, L, cur, list(new), El, dist)
            self.placement_host[L] = list(new)
            self.placement[L] = torch.tensor(new, dtype=torch.int32, device=self.device)
            store.expert_placement[L] = list(new)
            changed += 1
            moved_total += moved
        self.moves_done += moved_total
        return {"layers": changed, "moved": moved_total}

    def _move_experts(self, store, optimizer, L: int, cur, new, El: int, dist) -> None:
        """Experts of layer ``L`` change slots: ``cur[e]`` / ``new[e]`` = global slot (owner * El + local slot) of expert ``e`` before /
        after.  Master weights, work weights and optimizer state of every moved expert travel in ONE all-to-all of bytes over the
        expert group, which every rank of the group enters (with empty parts where it has nothing to move): point-to-point batches
        entered by only some of the ranks stalled on four GPUs.  Moves inside a rank are copies; nothing is overwritten before every
        outgoing part has been packed."""
        b = store.buckets.get(f"layer{L}.experts")
        if b is None:
            return
        tensors = [b.master]
        if b.work is not None and b.work is not b.master:
            tensors.append(b.work)
        st = optimizer.state.get(b.name) if hasattr(optimizer, "state") else None
        for t in (st or {}).values():
            tensors.append(t)
        n_master = b.master.numel()
        world, rank = self.ep, self.rank
        send_parts = [[] for _ in range(world)]      # per destination rank: byte views, in (expert, slot, tensor) order
        recv_specs = [[] for _ in range(world)]      # per source rank: (tensor, first, last) in the same order
        local = []
        for e in range(len(cur)):
            if cur[e] == new[e]:
                continue
            src_r, src_s, dst_r, dst_s = cur[e] // El, cur[e] % El, new[e] // El, new[e] % El
            for sl in b.slots:
                per = sl.numel // El
                for t in tensors:
                    div = n_master // t.numel() if t.numel() < n_master else 1   # group scales: one per 32 / 128 elements
                    a0, a1 = (sl.offset + src_s * per) // div, (sl.offset + (src_s + 1) * per) // div
                    d0, d1 = (sl.offset + dst_s * per) // div, (sl.offset + (dst_s + 1) * per) // div
                    if rank == src_r and rank == dst_r:
                        local.append((t, d0, d1, t[a0:a1].clone()))
                    elif rank == src_r:
                        send_parts[dst_r].append(t[a0:a1].contiguous().view(torch.uint8))
                    elif rank == dst_r:
                        recv_specs[src_r].append((t, d0, d1))
        dev = b.master.device
        in_splits = [int(sum(p.numel() for p in parts)) for parts in send_parts]
        out_splits = [int(sum((d1 - d0) * t.element_size() for t, d0, d1 in specs)) for specs in recv_specs]
        flat = [p for parts in send_parts for p in parts]
        send = torch.cat(flat) if flat else torch.empty(0, dtype=torch.uint8, device=dev)
        recv = torch.empty(sum(out_splits), dtype=torch.uint8, device=dev)
        group = getattr(self.comm.base, "group", None)
        dist.all_to_all_single(recv, send, out_splits, in_splits, group=group)
        at = 0
        for specs in recv_specs:
            for t, d0, d1 in specs:
                n = (d1 - d0) * t.element_size()
                t[d0:d1].copy_(recv[at:at + n].view(t.dtype))
                at += n
        for t, d0, d1, buf in local:   # only now: a slot's previous occupant has been packed or copied out above
            t[d0:d1].copy_(buf)

    # ------------------------------------------------------------------ balancing
    def dropped_rows(self) -> int:
        """Token copies dropped on this rank in the last step because an expert group overflowed the receive buffer."""
        return int(sum(int(v.item()) for v in self.last_overflow.values()))

    def imbalance(self) -> float:
        """max over layers of (busiest rank's tokens / mean rank tokens) in the last step (counts are in placed order)."""
        worst = 1.0
        for c in self.last_global_counts.values():
            per_rank = c.view(self.ep, -1).sum(1).float()
            worst = max(worst, float(per_rank.max() / per_rank.mean().clamp_min(1)))
        return worst

"""Expert parallelism through the library all-to-all: the portable form (any backend: gloo on CPU, NCCL), used by the PyTorch
reference backend and as the oracle of the peer-memory kernels in :mod:`surogate_b200.parallel.ep`.

Forward of one MoE layer on rank r of an expert group of size ``ep`` (``El = E / ep`` experts per rank):

1. the local permutation has sorted this rank's ``N * K`` token copies by global expert; rows for expert e are contiguous;
2. ``dispatch``: ranks exchange per-expert counts, then the rows (variable-split all-to-all); received rows arrive ordered
   [source rank][local expert] and are regrouped to [local expert][source rank], which is what the grouped GEMM wants;
3. ``combine``: the inverse regrouping and the inverse all-to-all bring every expert output back to the row its token copy
   came from.

Backward uses the same two exchanges in the opposite roles.  Sizes are read on the host (one small sync per exchange): this
path is for correctness and for machines without peer-mapped memory, not for speed.

Least-loaded balancing per step (``spill_threshold > 0``): when the busiest rank's routed rows exceed ``spill_threshold`` x the
mean, the LPT planner of the host runtime (``csrc/host/lpt_planner.cpp``) cuts the row ranges of overloaded experts into chunks and
hands chunks to less loaded ranks.  A helper rank then hosts extra expert slots for this layer and this step: the rows of a chunk are
dispatched to the helper instead of the owner, the owner ships that expert's weights to the helper (``extend_weights``, one
all-to-all per projection), the helper's grouped GEMM runs native and foreign slots alike, and in backward the helper returns the
foreign experts' weight gradients to their owners (``return_weight_grads``), where they are added to the owner's own.  The math is
unchanged: losses and gradients equal the unspilled run (``tests/test_multiprocess_cpu.py``).

Parity: csrc/src/runtime/ep/ep_strategy.cpp:621-856 (split exchange + grouped send / recv), :468-503 (LLEP plan),
csrc/src/runtime/ep/weight_transfer.cpp:148-445 (foreign expert weights and gradient return).
"""
from __future__ import annotations

from typing import List

import torch


class _RecvPlan:
    """What the experts' owner sees: rows grouped by local expert (``offsets`` [El + 1], ``counts`` [El])."""

    def __init__(self, local, offsets, counts, send_splits: List[int], recv_splits: List[int], regroup: torch.Tensor, x_shape):
        self.local = local                      # the sender-side permutation plan (moe_permute's)
        self.offsets, self.counts = offsets, counts
        self.send_splits, self.recv_splits = send_splits, recv_splits
        self.regroup = regroup                  # received order -> expert-major order
        self.num_tokens, self.top_k, self.num_experts, self.x_shape = local.num_tokens, local.top_k, counts.numel(), x_shape
        self.ep = self                          # marks an expert-parallel plan for ops that look for one
        self.sorted_src = local.sorted_src
        self.send_idx = None                    # spilled steps: order in which this rank's permuted rows leave ([dest][slot])
        self.foreign = []                       # spilled steps: [(global expert, owner rank, helper rank)] in slot order per helper
        self.w_ext = {}                         # role -> weights of native + foreign slots on this rank (kept from forward for backward)


class AllToAllExpertParallel:
    def __init__(self, comm, ep_size: int, device, spill_threshold: float = 0.0, spill_capacity: float = 1.1, spill_min_rows: int = 1):
        if comm.world != ep_size:
            raise ValueError(f"the expert group has {comm.world} ranks but ep_size is {ep_size}")
        self.comm, self.ep, self.rank, self.device = comm, ep_size, comm.rank, device
        self.spill_threshold, self.spill_capacity, self.spill_min_rows = spill_threshold, spill_capacity, spill_min_rows
        self.spilled_layers = 0
        self.last_global_counts = {}
        self.placement = {}
        self.moves_done = 0

    # -- helpers
    def _exchange(self, rows: torch.Tensor, send_splits: List[int], recv_splits: List[int]) -> torch.Tensor:
        out = torch.empty((sum(recv_splits),) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
        self.comm.all_to_all_single(out, rows.contiguous(), recv_splits, send_splits)
        return out

    def place(self, layer, topk_idx, counts):
        return topk_idx, counts

    # -- forward
    def dispatch(self, ctx, xp: torch.Tensor, plan):
        E = plan.counts.numel()
        El = E // self.ep
        counts = plan.counts.to(torch.int64)
        all_counts = torch.empty(self.ep * E, dtype=torch.int64, device=xp.device)        # [source][expert]
        gathered = list(all_counts.view(self.ep, E).unbind(0))
        import torch.distributed as dist

        dist.all_gather(gathered, counts.contiguous(), group=self.comm.group)
        table = all_counts.view(self.ep, E)
        if self.spill_threshold > 0 and getattr(ctx, "lora", None) is None:
            spilled = self._dispatch_spilled(ctx, xp, plan, table, E, El)
            if spilled is not None:
                return spilled
        mine = table[:, self.rank * El:(self.rank + 1) * El]                              # [source, local expert] rows I receive
        send_splits = counts.view(self.ep, El).sum(1).tolist()
        recv_splits = mine.sum(1).tolist()
        recv = self._exchange(xp, send_splits, recv_splits)
        # regroup [source][expert] -> [expert][source]
        m = mine.tolist()
        src_start = [0]
        for s in range(self.ep):
            src_start.append(src_start[-1] + sum(m[s]))
        idx = []
        for e in range(El):
            for s in range(self.ep):
                a = src_start[s] + sum(m[s][:e])
                idx.append(torch.arange(a, a + m[s][e], device=xp.device))
        regroup = torch.cat(idx) if idx else torch.zeros(0, dtype=torch.long, device=xp.device)
        per_expert = mine.sum(0).to(torch.int32)
        offsets = torch.zeros(El + 1, dtype=torch.int32, device=xp.device)
        offsets[1:] = torch.cumsum(per_expert, 0)
        if ctx.layer is not None and getattr(ctx, "phase", "fwd") == "fwd":
            self.last_global_counts[ctx.layer] = table.sum(0)
        return recv[regroup], _RecvPlan(plan, offsets, per_expert, send_splits, recv_splits, regroup, plan.x_shape)

    # -- least-loaded balancing: token ranges of overloaded experts go to helper ranks for this step
    def _dispatch_spilled(self, ctx, xp, plan, table, E, El):
        from ..ops import host

        t = table.tolist()                                   # [source][expert]
        g = [sum(t[s][e] for s in range(self.ep)) for e in range(E)]
        lp = host().compute_lpt_plan(g, self.ep, float(self.spill_threshold), float(self.spill_capacity), int(self.spill_min_rows))
        if not lp["uses_lpt"]:
            return None
        # slots of every rank: its native experts, then the foreign experts it helps with (ascending expert id)
        chunks = {}                                          # (helper rank, expert) -> [(a, b)] ranges of the expert's global row order
        for e, parts in enumerate(lp["assignments"]):
            for h, a, b in parts:
                if b > a:
                    chunks.setdefault((h, e), []).append((a, b))
        slots = []
        for h in range(self.ep):
            native = list(range(h * El, (h + 1) * El))
            foreign = sorted(e for (hh, e) in chunks if hh == h and e // El != h)
            slots.append(native + foreign)
        first = [[sum(t[r][e] for r in range(s)) for e in range(E)] for s in range(self.ep)]       # global position of source s's first row of e

        def rows_from(s, h, e):                              # [(lo, hi)] ranges, relative to source s's rows of expert e, that go to helper h
            out = []
            for a, b in chunks.get((h, e), []):
                lo, hi = max(a, first[s][e]) - first[s][e], min(b, first[s][e] + t[s][e]) - first[s][e]
                if hi > lo:
                    out.append((lo, hi))
            return out

        route = [[[sum(hi - lo for lo, hi in rows_from(s, h, e)) for e in slots[h]] for h in range(self.ep)] for s in range(self.ep)]
        me = self.rank
        my_start = [0]
        for e in range(E):
            my_start.append(my_start[-1] + t[me][e])
        idx = []
        for h in range(self.ep):
            for e in slots[h]:
                for lo, hi in rows_from(me, h, e):
                    idx.append(torch.arange(my_start[e] + lo, my_start[e] + hi, device=xp.device))
        send_idx = torch.cat(idx) if idx else torch.zeros(0, dtype=torch.long, device=xp.device)
        assert send_idx.numel() == xp.shape[0], "every routed row leaves exactly once"
        send_splits = [sum(route[me][h]) for h in range(self.ep)]
        recv_splits = [sum(route[s][me]) for s in range(self.ep)]
        recv = self._exchange(xp[send_idx], send_splits, recv_splits)
        S = len(slots[me])
        src_start = [0]
        for s in range(self.ep):
            src_start.append(src_start[-1] + recv_splits[s])
        ridx = []
        for k in range(S):
            for s in range(self.ep):
                a = src_start[s] + sum(route[s][me][:k])
                ridx.append(torch.arange(a, a + route[s][me][k], device=xp.device))
        regroup = torch.cat(ridx) if ridx else torch.zeros(0, dtype=torch.long, device=xp.device)
        per_slot = torch.tensor([sum(route[s][me][k] for s in range(self.ep)) for k in range(S)], dtype=torch.int32, device=xp.device)
        offsets = torch.zeros(S + 1, dtype=torch.int32, device=xp.device)
        offsets[1:] = torch.cumsum(per_slot, 0)
        rp = _RecvPlan(plan, offsets, per_slot, send_splits, recv_splits, regroup, plan.x_shape)
        rp.send_idx = send_idx
        rp.foreign = [(e, e // El, h) for h in range(self.ep) for e in slots[h][El:]]
        rp.El = El
        if ctx.layer is not None and getattr(ctx, "phase", "fwd") == "fwd":
            self.last_global_counts[ctx.layer] = table.sum(0)
            self.spilled_layers += 1
        return recv[regroup], rp

    def _weights_all_to_all(self, parts_for, shapes_from, like: torch.Tensor):
        """``parts_for[r]`` = list of tensors this rank sends to rank r; ``shapes_from[r]`` = list of shapes it receives from rank r.
        One all-to-all of flattened elements (every rank of the group enters, also with nothing to send)."""
        send = [p.reshape(-1) for r in range(self.ep) for p in parts_for[r]]
        flat = torch.cat(send) if send else like.new_zeros(0)
        in_splits = [int(sum(p.numel() for p in parts_for[r])) for r in range(self.ep)]
        out_splits = [int(sum(int(torch.Size(sh).numel()) for sh in shapes_from[r])) for r in range(self.ep)]
        out = like.new_empty(sum(out_splits))
        self.comm.all_to_all_single(out, flat.contiguous(), out_splits, in_splits)
        got, at = [], 0
        for r in range(self.ep):
            for sh in shapes_from[r]:
                n = int(torch.Size(sh).numel())
                got.append(out[at:at + n].view(sh))
                at += n
        return got

    def extend_weights(self, ctx, role: str, w_local: torch.Tensor, plan: _RecvPlan) -> torch.Tensor:
        """Weights of this rank's slots for a spilled step: its own experts followed by the foreign experts it helps with, shipped by
        their owners.  Collective over the expert group; kept on the plan for backward."""
        if not plan.foreign and plan.send_idx is None:
            return w_local
        cached = plan.w_ext.get(role)
        if cached is not None:
            return cached
        El, me = plan.El, self.rank
        parts_for = [[w_local[e - me * El] for (e, o, h) in plan.foreign if o == me and h == r] for r in range(self.ep)]
        shapes_from = [[tuple(w_local.shape[1:]) for (e, o, h) in plan.foreign if h == me and o == r] for r in range(self.ep)]
        got = self._weights_all_to_all(parts_for, shapes_from, w_local)
        mine = [(e, o) for (e, o, h) in plan.foreign if h == me]          # slot order: ascending expert id
        by_owner = sorted(range(len(mine)), key=lambda i: (mine[i][1], mine[i][0]))   # arrival order: by owner rank, then expert id
        ordered = [None] * len(mine)
        for pos, i in enumerate(by_owner):
            ordered[i] = got[pos]
        w_ext = torch.cat([w_local] + [x.unsqueeze(0) for x in ordered]) if ordered else w_local
        assert w_ext.shape[0] == int(plan.counts.numel()), (role, tuple(w_ext.shape), int(plan.counts.numel()), plan.foreign, me, El)
        plan.w_ext[role] = w_ext
        return w_ext

    def return_weight_grads(self, ctx, role: str, dw_foreign, plan: _RecvPlan, like: torch.Tensor):
        """``dw_foreign``: this helper's weight gradients of its foreign slots (slot order).  Returns [(local expert index, gradient)]
        contributions of other ranks to this rank's own experts.  Collective over the expert group."""
        El, me = plan.El, self.rank
        mine = [(e, o) for (e, o, h) in plan.foreign if h == me]
        parts_for = [[dw_foreign[i] for i, (e, o) in enumerate(mine) if o == r] for r in range(self.ep)]
        incoming = [[(e, h) for (e, o, h) in plan.foreign if o == me and h == r] for r in range(self.ep)]
        shapes_from = [[tuple(like.shape[1:]) for _ in incoming[r]] for r in range(self.ep)]
        got = self._weights_all_to_all(parts_for, shapes_from, like)
        out, at = [], 0
        for r in range(self.ep):
            for e, h in incoming[r]:
                out.append((e - me * El, got[at]))
                at += 1
        return out

    def _back(self, rows: torch.Tensor, plan: _RecvPlan) -> torch.Tensor:
        ungrouped = torch.empty_like(rows)
        ungrouped[plan.regroup] = rows
        back = self._exchange(ungrouped, plan.recv_splits, plan.send_splits)
        if plan.send_idx is not None:           # spilled step: the rows left in [dest][slot] order, put them back in permuted order
            out = torch.empty_like(back)
            out[plan.send_idx] = back
            return out
        return back

    def combine(self, ctx, y: torch.Tensor, plan: _RecvPlan) -> torch.Tensor:
        """Expert outputs (forward) or the experts' input gradients (backward of dispatch) return to the token copies' rows."""
        return self._back(y, plan)

    def dispatch_backward(self, ctx, dy: torch.Tensor, plan: _RecvPlan) -> torch.Tensor:
        """Gradients of the returned rows travel to the experts' owner, in the order the forward delivered the inputs."""
        recv = self._exchange(dy if plan.send_idx is None else dy[plan.send_idx], plan.send_splits, plan.recv_splits)
        return recv[plan.regroup]

    # -- statistics used by the trainer
    def dropped_rows(self) -> int:
        return 0

    def imbalance(self) -> float:
        worst = 1.0
        for c in self.last_global_counts.values():
            per_rank = c.view(self.ep, -1).sum(1).float()
            worst = max(worst, float(per_rank.max() / per_rank.mean().clamp_min(1)))
        return worst

    def rebalance(self, *a, **k):
        return {"layers": 0, "moved": 0}

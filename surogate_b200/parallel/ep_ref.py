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

Parity: csrc/src/runtime/ep/ep_strategy.cpp:621-856 (split exchange + grouped send / recv).
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


class AllToAllExpertParallel:
    def __init__(self, comm, ep_size: int, device):
        if comm.world != ep_size:
            raise ValueError(f"the expert group has {comm.world} ranks but ep_size is {ep_size}")
        self.comm, self.ep, self.rank, self.device = comm, ep_size, comm.rank, device
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

    def _back(self, rows: torch.Tensor, plan: _RecvPlan) -> torch.Tensor:
        ungrouped = torch.empty_like(rows)
        ungrouped[plan.regroup] = rows
        return self._exchange(ungrouped, plan.recv_splits, plan.send_splits)

    def combine(self, ctx, y: torch.Tensor, plan: _RecvPlan) -> torch.Tensor:
        """Expert outputs (forward) or the experts' input gradients (backward of dispatch) return to the token copies' rows."""
        return self._back(y, plan)

    def dispatch_backward(self, ctx, dy: torch.Tensor, plan: _RecvPlan) -> torch.Tensor:
        """Gradients of the returned rows travel to the experts' owner, in the order the forward delivered the inputs."""
        recv = self._exchange(dy, plan.send_splits, plan.recv_splits)
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

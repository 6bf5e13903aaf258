"""The expert-parallel x data-parallel mesh: ``world = dp x ep`` with ``ep_rank = rank % ep`` and ``dp_index = rank // ep``.

* the EXPERT GROUP of a rank is the ``ep`` consecutive ranks of its data-parallel replica: token dispatch / combine and the
  gathering of expert weights for export happen inside it;
* the EXPERT DATA-PARALLEL GROUP of a rank is the ``dp`` ranks that hold the same experts (same ``ep_rank`` in every replica):
  expert gradients are summed over it, and over nothing else;
* every other parameter is data-parallel (or ZeRO-sharded) over the whole world, as without experts.

Every rank creates every group (``torch.distributed.new_group`` is collective over the world) and keeps its own two.

Parity: csrc/src/utilities/comm.cpp:515-580 (EP / DP sub-communicators of the reference).
"""
from __future__ import annotations

from typing import Optional, Tuple


def build_ep_mesh(world_comm, ep_size: int) -> Tuple[Optional[object], Optional[object]]:
    """(communicator of this rank's expert group, communicator of its expert data-parallel group); (None, None) when the expert
    group is the whole world (``dp = 1``)."""
    world, rank = world_comm.world, world_comm.rank
    if ep_size <= 1 or ep_size >= world:
        return None, None
    if world % ep_size:
        raise ValueError(f"ep_size={ep_size} does not divide the {world} ranks")
    import torch.distributed as dist

    from .dist import TorchComm

    dp = world // ep_size
    ep_comm = edp_comm = None
    for d in range(dp):                       # expert groups: consecutive ranks
        ranks = list(range(d * ep_size, (d + 1) * ep_size))
        g = dist.new_group(ranks)
        if rank in ranks:
            ep_comm = TorchComm(g)
    for e in range(ep_size):                  # expert data-parallel groups: same ep_rank in every replica
        ranks = [e + d * ep_size for d in range(dp)]
        g = dist.new_group(ranks)
        if rank in ranks:
            edp_comm = TorchComm(g)
    return ep_comm, edp_comm

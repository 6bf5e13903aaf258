"""Process-per-GPU distributed context over ``torch.distributed`` (NCCL on GPUs, gloo on CPU).

``TorchComm`` is the library-collective implementation of the small interface the
parameter store needs (all_gather / reduce_scatter / all_reduce on flat buffers).
It is the *baseline* data plane; :mod:`surogate_b200.parallel.symm` provides the
same interface with hand-written peer-memory kernels.

Parity: csrc/src/utilities/comm.{h,cpp} (NCCLCommunicator) — the thread-per-GPU
launcher, shared launch-queue throttling and memcpy emulations of the reference are
not needed with one process per GPU on an NVSwitch fabric.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class DistInfo:
    rank: int = 0
    world: int = 1
    local_rank: int = 0
    backend: str = "none"

    @property
    def is_main(self) -> bool:
        return self.rank == 0


def init_distributed(backend: Optional[str] = None, timeout_s: int = 600) -> DistInfo:
    """Initialise from torchrun-style environment variables; a no-op for single-process runs."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return DistInfo()
    rank = int(os.environ["RANK"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if backend == "nccl":
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return DistInfo(rank, world, local_rank, backend)


_OPS = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}


class TorchComm:
    """Collectives on flat tensors through torch.distributed (NCCL / gloo)."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.backend = dist.get_backend(group)

    def all_gather(self, shard: torch.Tensor, full: torch.Tensor, async_op: bool = False):
        if self.backend == "gloo":
            parts = list(full.view(self.world, -1).unbind(0))
            return dist.all_gather(parts, shard.contiguous(), group=self.group, async_op=async_op)
        return dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group, async_op=async_op)

    def reduce_scatter(self, full: torch.Tensor, shard: torch.Tensor, async_op: bool = False, average: bool = False):
        if self.backend == "gloo":
            tmp = full.clone()
            dist.all_reduce(tmp, group=self.group)
            n = shard.numel()
            shard.copy_(tmp[self.rank * n:(self.rank + 1) * n])
            if average:
                shard.div_(self.world)
            return None
        op = dist.ReduceOp.AVG if average else dist.ReduceOp.SUM
        return dist.reduce_scatter_tensor(shard, full, op=op, group=self.group, async_op=async_op)

    def all_reduce(self, t: torch.Tensor, op: str = "sum", async_op: bool = False):
        if op == "avg":
            if self.backend == "gloo":
                w = dist.all_reduce(t, group=self.group)
                t.div_(self.world)
                return None
            return dist.all_reduce(t, op=dist.ReduceOp.AVG, group=self.group, async_op=async_op)
        return dist.all_reduce(t, op=_OPS[op], group=self.group, async_op=async_op)

    def all_to_all_single(self, out: torch.Tensor, inp: torch.Tensor, out_splits=None, in_splits=None, async_op: bool = False):
        return dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group, async_op=async_op)

    def broadcast(self, t: torch.Tensor, src: int = 0):
        return dist.broadcast(t, src=dist.get_global_rank(self.group, src) if self.group is not None else src, group=self.group)

    def barrier(self):
        dist.barrier(group=self.group)

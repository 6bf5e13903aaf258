"""Collectives over symmetric (peer-mapped) memory, executed by this framework's own kernels.

Plumbing (allocation of the symmetric arena and exchange of the mapping handles between the ranks'
processes) goes through ``torch.distributed._symmetric_memory``; every byte that crosses NVLink afterwards
is moved by the kernels in ``csrc/comm_kernels.cu``: a rank's kernel loads directly from its peers' arenas.

``SymmComm`` offers the same small interface as :class:`~surogate_b200.parallel.dist.TorchComm`
(``all_gather`` / ``reduce_scatter`` / ``all_reduce`` / ``barrier``) plus ``create_arena`` so that the
parameter store can place master shards and gradient buckets where peers can reach them.  Operations whose
buffers are not in the arena fall back to the library communicator.

Ordering rules the kernels rely on:
* a flag barrier precedes every reduce-scatter (all ranks have finished writing the bucket);
* ``fence()`` (a barrier) is called by the trainer before the optimizer changes the master shards and after it,
  so gathers never observe a half-updated shard and no shard is overwritten while a peer still reads it.
"""
from __future__ import annotations

import os

from typing import List, Optional

import torch

# signal-pad channels (8 uint32 words each).  A channel is only ever used from ONE stream, so its epochs are
# observed in program order; mixing streams on one channel would let a later epoch satisfy an earlier barrier.
SLOT_MAIN = 0  # fences on the compute stream
SLOT_SIDE = 8  # barriers that precede collectives on the communication stream
SLOT_ALLREDUCE = 16  # flag exchange inside the small all-reduce (compute stream)
PAD_WORDS = 256
SCRATCH_FLOATS = 2 * 1024  # two alternating regions for the one-shot small all-reduce


class _Work:
    """Completion handle compatible with torch.distributed work objects: wait() orders the current stream after the op."""

    def __init__(self, event: torch.cuda.Event):
        self.event = event

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)


_ARENAS_ALIVE: List["Arena"] = []


class Arena:
    def __init__(self, tensor: torch.Tensor, peer_bases: List[int], mc_base: int):
        self.tensor = tensor  # uint8 view of the whole local arena
        self.peer_bases = peer_bases
        self.mc_base = mc_base
        self.base = tensor.data_ptr()
        self.nbytes = tensor.numel()
        self.cursor = 0

    def take(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        es = torch.empty((), dtype=dtype).element_size()
        start = (self.cursor + 255) // 256 * 256
        end = start + numel * es
        if end > self.nbytes:
            raise MemoryError(f"symmetric arena exhausted ({end} > {self.nbytes} bytes)")
        self.cursor = end
        return self.tensor[start:end].view(dtype)

    def offset_of(self, t: torch.Tensor) -> Optional[int]:
        off = t.data_ptr() - self.base
        return off if 0 <= off < self.nbytes else None


class SymmComm:
    def __init__(self, base, device, symm_mod, group):
        self.base = base
        self.rank, self.world = base.rank, base.world
        self.device = device
        self._symm = symm_mod
        self._group = group
        from ..ops import ext

        self.ext = ext()
        self.err = self.ext.error_flag_tensor()
        self.stream = torch.cuda.Stream(device=device)
        self.arena: Optional[Arena] = None
        self.epochs = {SLOT_MAIN: 0, SLOT_SIDE: 0}
        self.ar_epoch = 0
        self.max_blocks = 96
        self.wait_budget_s = float(os.environ.get("SUROGATE_WAIT_BUDGET_S", "20"))   # every cross-GPU wait gives up after this long and raises the error flag
        self.use_multimem = False
        # control block: signal pad + small all-reduce scratch, in its own small symmetric allocation
        self.ctrl = self._alloc_symmetric(PAD_WORDS * 4 + SCRATCH_FLOATS * 4)
        self.ctrl.tensor.zero_()
        torch.cuda.synchronize(device)
        base.barrier()

    # ------------------------------------------------------------------ set-up
    @staticmethod
    def create(base, device) -> Optional["SymmComm"]:
        if base is None or base.world < 2 or base.world > 8 or device.type != "cuda":
            return None
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        group = base.group if base.group is not None else dist.group.WORLD
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:  # noqa: BLE001  (newer releases enable groups implicitly)
            pass
        return SymmComm(base, device, symm_mem, group)

    def _alloc_symmetric(self, nbytes: int) -> Arena:
        nbytes = (nbytes + 4095) // 4096 * 4096
        t = self._symm.empty(nbytes, dtype=torch.uint8, device=self.device)
        hdl = self._symm.rendezvous(t, group=self._group)
        bases = [int(p) for p in hdl.buffer_ptrs]
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        a = Arena(t, bases, mc)
        a.handle = hdl
        # Peer-mapped blocks are kept until the process ends: a run that released such buffers and allocated new ones right afterwards
        # stalled (both ranks waited on each other until the job was killed), most likely because the new block reused the address and
        # the cached peer mappings of the old one.  A trainer that is rebuilt inside one process (out-of-memory retry with a smaller
        # micro-batch, a second model in a benchmark) therefore adds arenas instead of replacing them.
        _ARENAS_ALIVE.append(a)
        return a

    def create_arena(self, nbytes: int) -> Arena:
        self.arena = self._alloc_symmetric(nbytes)
        return self.arena

    # ------------------------------------------------------------------ primitives
    def _barrier(self, channel: int):
        self.epochs[channel] += 1
        self.ext.symm_barrier(self.ctrl.peer_bases, self.rank, self.epochs[channel] & 0x7FFFFFFF, channel, self.err, self.wait_budget_s)

    def barrier(self):
        self._barrier(SLOT_MAIN)

    def fence(self):
        """Device-side barrier on the compute stream (no host synchronisation)."""
        self._barrier(SLOT_MAIN)

    def _side(self):
        """Enter the communication stream, ordered after everything queued so far on the current stream."""
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.stream.wait_event(ev)
        return torch.cuda.stream(self.stream)

    def _done(self, async_op: bool):
        ev = torch.cuda.Event()
        ev.record(self.stream)
        w = _Work(ev)
        if not async_op:
            w.wait()
            return None
        return w

    # ------------------------------------------------------------------ collectives
    def reduce_scatter(self, full: torch.Tensor, shard: torch.Tensor, async_op: bool = False, average: bool = False, sumsq_out=None,
                       accumulate: bool = False):
        off = self.arena.offset_of(full) if self.arena is not None else None
        if off is None or full.dtype != torch.bfloat16:
            return self.base.reduce_scatter(full, shard, async_op=async_op, average=average)
        scale = 1.0 / self.world if average else 1.0
        with self._side():
            self._barrier(SLOT_SIDE)
            if self.use_multimem and self.arena.mc_base and not accumulate:
                self.ext.reduce_scatter_multimem(self.arena.mc_base, off, shard.numel(), self.rank, scale, shard, sumsq_out, self.max_blocks)
            else:
                self.ext.reduce_scatter_fused(self.arena.peer_bases, off, shard.numel(), self.rank, scale, shard, accumulate, sumsq_out, self.max_blocks)
            shard.record_stream(self.stream)
        return self._done(async_op)

    def all_gather(self, shard: torch.Tensor, full: torch.Tensor, async_op: bool = False, out_fp8=None, scale=None, segment=None):
        off = self.arena.offset_of(shard) if self.arena is not None else None
        if off is None or shard.dtype != torch.bfloat16:
            return self.base.all_gather(shard, full, async_op=async_op)
        lo, hi = segment if segment is not None else (0, shard.numel() * self.world)
        with self._side():
            self.ext.all_gather_fused(self.arena.peer_bases, off, shard.numel(), lo, hi, full, out_fp8, scale, self.max_blocks)
            if full is not None:
                full.record_stream(self.stream)
            if scale is not None:
                scale.record_stream(self.stream)
            if out_fp8 is not None:
                out_fp8.record_stream(self.stream)
        return self._done(async_op)

    def all_gather_bytes(self, shard_u8: torch.Tensor, full_u8: torch.Tensor, arena: "Arena", segment, async_op: bool = False):
        """Pull bytes ``[lo, hi)`` of the gathered bucket from the peers' byte shards (already-quantised FP8 weights: one byte per
        weight crosses NVLink instead of two).  The gather kernel moves 16-byte vectors and never looks inside them, so the byte
        buffers are passed as bf16 pairs with every count halved; ``lo`` / ``hi`` / the shard size must be multiples of 16."""
        off = arena.offset_of(shard_u8)
        lo, hi = segment
        assert off is not None and shard_u8.dtype == torch.uint8 and full_u8.dtype == torch.uint8
        assert lo % 16 == 0 and hi % 16 == 0 and shard_u8.numel() % 16 == 0 and off % 16 == 0, "byte gather: 16-byte granularity"
        with self._side():
            self.ext.all_gather_fused(arena.peer_bases, off, shard_u8.numel() // 2, lo // 2, hi // 2, full_u8.view(torch.bfloat16), None, None, self.max_blocks)
            full_u8.record_stream(self.stream)
        return self._done(async_op)

    def all_gather_from_host(self, host_shard: torch.Tensor, stage: torch.Tensor, full: torch.Tensor, async_op: bool = False):
        """ZeRO-3 gather of a shard that lives in pinned host memory: the H2D copy lands in a peer-visible arena slot, a
        device-side barrier says that every rank's copy has landed, then the gather kernel pulls the peers' slots.  All on
        the communication stream, so the PCIe copy and the NVLink pulls overlap the compute stream.  Callers alternate
        between two slots: the barrier of gather k+1 also proves that every peer finished pulling slot k."""
        off = self.arena.offset_of(stage)
        assert off is not None and stage.dtype == torch.bfloat16 and host_shard.numel() == stage.numel()
        with self._side():
            stage.copy_(host_shard, non_blocking=True)
            self._barrier(SLOT_SIDE)
            self.ext.all_gather_fused(self.arena.peer_bases, off, stage.numel(), 0, stage.numel() * self.world, full, None, None, self.max_blocks)
            full.record_stream(self.stream)
        return self._done(async_op)

    def all_reduce(self, t: torch.Tensor, op: str = "sum", async_op: bool = False):
        if t.dtype == torch.float32 and t.numel() <= 1024 and t.is_contiguous() and op in ("sum", "max", "avg"):
            self.ar_epoch += 1
            region = (self.ar_epoch & 1) * 1024 * 4
            self.ext.all_reduce_small(self.ctrl.peer_bases, self.ctrl.peer_bases, PAD_WORDS * 4 + region, t.view(-1), 1 if op == "max" else 0,
                                      self.rank, self.ar_epoch & 0x7FFFFFFF, SLOT_ALLREDUCE, self.err, self.wait_budget_s)
            if op == "avg":
                t.div_(self.world)
            return None
        return self.base.all_reduce(t, op=op, async_op=async_op)

    def __getattr__(self, name):  # everything else (all_to_all_single, broadcast, group ...) is the library communicator's
        return getattr(self.base, name)

"""Device memory handed out in stack order, and the registry behind the memory breakdown.

``DeviceStack`` owns one large device tensor and sub-allocates transients from it in LIFO order with the native bookkeeping
of ``csrc/host/memory_stack.cpp``: a phase (the LM-head chunk loop, a recomputed layer) opens a ``frame()``, takes its buffers
and releases them all at once when the frame closes.  A phase gets the same addresses every step, which is what a captured
CUDA graph needs, and nothing goes through the allocator in the hot loop.  The high-water mark and the per-name peaks say how
large the stack has to be.

``registry_for(trainer)`` fills a native ``AllocationRegistry`` with everything long-lived (weights, gradients, optimizer
state, host copies, symmetric arena, stack) by category and memory kind.

Parity: csrc/src/utilities/stack.h (DeviceMemoryStack), csrc/src/utilities/allocator.h (TensorAllocator, EAllocationType).
"""
from __future__ import annotations

import contextlib
import math
from typing import Dict, Optional, Sequence

import torch

ALIGN = 4096


class DeviceStack:
    def __init__(self, device, capacity_bytes: int = 0, name: str = "stack"):
        from ..ops import host

        self._host = host()
        self.device = torch.device(device)
        self.name = name
        self.buf: Optional[torch.Tensor] = None
        self.native = None
        self._base_off = 0
        if capacity_bytes > 0:
            self._reserve(capacity_bytes)

    # ------------------------------------------------------------------ storage
    def _reserve(self, capacity_bytes: int) -> None:
        cap = (int(capacity_bytes) + ALIGN - 1) // ALIGN * ALIGN
        self.buf = torch.empty(cap + ALIGN, dtype=torch.uint8, device=self.device)
        self._base_off = (-self.buf.data_ptr()) % ALIGN
        self.native = self._host.MemoryStack(self.buf.data_ptr() + self._base_off, cap, ALIGN)

    @property
    def capacity(self) -> int:
        return int(self.native.capacity) if self.native is not None else 0

    @property
    def used(self) -> int:
        return int(self.native.used) if self.native is not None else 0

    @property
    def high_water(self) -> int:
        return int(self.native.high_water) if self.native is not None else 0

    def can_grow(self) -> bool:
        """The backing tensor may be replaced only while nothing is allocated from it and no CUDA graph is being captured."""
        capturing = self.device.type == "cuda" and torch.cuda.is_current_stream_capturing()
        return self.used == 0 and not capturing

    # ------------------------------------------------------------------ allocation
    def alloc(self, shape: Sequence[int], dtype: torch.dtype, name: str = "") -> torch.Tensor:
        nbytes = max(1, math.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        need = (nbytes + ALIGN - 1) // ALIGN * ALIGN
        if self.native is None or self.used + need > self.capacity:
            if not self.can_grow():
                raise RuntimeError(f"device stack '{self.name}' is full ({self.used} of {self.capacity} bytes used) and cannot grow now: "
                                   f"'{name}' needs {need} bytes; live: {self.native.live() if self.native is not None else []}")
            self._reserve(max(need, 2 * self.capacity))
        addr = self.native.allocate(nbytes, name)
        off = addr - self.buf.data_ptr()
        return self.buf[off:off + nbytes].view(dtype).view(*shape)

    def fits(self, nbytes: int) -> bool:
        need = (nbytes + ALIGN - 1) // ALIGN * ALIGN
        return (self.native is not None and self.used + need <= self.capacity) or self.can_grow()

    @contextlib.contextmanager
    def frame(self):
        cp = self.native.checkpoint() if self.native is not None else 0
        grown_from = self.native
        try:
            yield self
        finally:
            if self.native is grown_from and self.native is not None:
                self.native.restore(cp)
            elif self.native is not None:  # the stack was replaced by a larger one inside the frame (it was empty before)
                self.native.restore(0)

    def stats(self) -> Dict[str, object]:
        if self.native is None:
            return {"capacity": 0, "used": 0, "high_water": 0, "allocations": 0, "peak_by_name": {}}
        return {"capacity": self.capacity, "used": self.used, "high_water": self.high_water, "allocations": int(self.native.allocations),
                "peak_by_name": dict(self.native.peak_by_name())}


def _kind(t: torch.Tensor) -> str:
    if t.device.type == "cuda":
        return "device"
    return "pinned" if t.is_pinned() else "host"


def registry_for(trainer):
    """Native registry of the trainer's long-lived allocations: parameter masters, work copies, gradients, host copies, optimizer
    state, LoRA adapters, the symmetric arena and the transient stack."""
    from ..ops import host

    reg = host().AllocationRegistry()
    seen = set()

    def add(name: str, category: str, t) -> None:
        if not torch.is_tensor(t) or t.numel() == 0:
            return
        key = (t.untyped_storage().data_ptr(), t.untyped_storage().nbytes())
        if key in seen:
            return
        seen.add(key)
        reg.record(name, category, _kind(t), t.numel() * t.element_size())

    arena = getattr(trainer.store, "arena", None)
    if arena is not None and torch.is_tensor(getattr(arena, "tensor", None)):
        add("symmetric_arena", "arena", arena.tensor)
    for b in trainer.store.buckets.values():
        add(f"{b.name}.master", "weights_master", b.master)
        if b.work is not None and b.work is not b.master:
            add(f"{b.name}.work", "weights_work", b.work)
        for attr, cat in (("work_host", "weights_host_copy"), ("work_next", "weights_host_copy"), ("grad", "gradients")):
            add(f"{b.name}.{attr}", cat, getattr(b, attr, None))
    for bname, st in getattr(trainer.optimizer, "state", {}).items():
        for k, t in st.items():
            add(f"{bname}.opt.{k}", "optimizer_state", t)
    lora = getattr(trainer, "lora", None)
    for n, t in (lora.named_tensors() if lora is not None and hasattr(lora, "named_tensors") else []):
        add(f"lora.{n}", "lora", t)
    stack = getattr(trainer.backend, "stack", None)
    if stack is not None and stack.buf is not None:
        add("transient_stack", "stack", stack.buf)
    return reg

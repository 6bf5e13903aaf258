"""Parameter / gradient storage in flat per-layer buckets, with ZeRO-1/2/3 sharding.

Every layer (and each of embedding / final norm / LM head) owns one contiguous
*bucket*.  A bucket is the concatenation of its parameters, each starting on a
256-byte boundary, padded so that it splits evenly across ranks.  Rank ``r``
owns elements ``[r*S, (r+1)*S)`` of every bucket (master weights, optimizer
state).  Consequences:

* a ZeRO-3 weight gather and a gradient reduce-scatter are each ONE contiguous
  collective per layer, and the element-wise optimizer runs on the flat shard;
* parameters are views into the gathered bucket, gradients views into the
  bucket-sized gradient buffer that weight-gradient GEMMs accumulate into.

Sharding levels (``zero_level``): 0 = replicated + all-reduce; 1 = gradients
reduce-scattered at the last micro-step, optimizer state and master weights
sharded, updated weights all-gathered once per step; 2 = additionally the
bucket-sized gradient buffers are transient (reduce-scatter every micro-step
into an fp32 shard accumulator); 3 = additionally the gathered work weights are
transient: gathered per layer one layer ahead of use and released after use
(or kept for the rest of the step when ``keep_gathered`` and memory allow).

Parity: csrc/src/runtime/dsl/dsl_param_store, dsl_grad_store.cpp:457-678
(notify_block / scatter_reduce_layer), dsl_weight_manager.cpp:779-1076 (gather_block).
"""
from __future__ import annotations

import os

import math
import zlib
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple

import torch

from ..dsl.compiler import CompiledModel, ParamEntry

ALIGN_ELEMS = 128
FP8_SHARDS_DEFAULT = "1"   # quantise-then-gather of ZeRO-3 FP8 weights (SUROGATE_FP8_SHARDS=0: peers pull bf16 and quantise on arrival)


@dataclass
class Slot:
    name: str
    offset: int
    numel: int
    shape: Tuple[int, ...]
    decay: bool
    entry: ParamEntry
    trainable: bool = True


class Bucket:
    def __init__(self, name: str, layer: Optional[int]):
        self.name = name
        self.layer = layer
        self.slots: List[Slot] = []
        self.numel = 0  # padded
        self.shard_numel = 0
        self.master: Optional[torch.Tensor] = None  # [shard_numel] (or full when world == 1 / level 0)
        self.work: Optional[torch.Tensor] = None  # [numel] gathered work weights (None when released)
        self.work_fp8: Optional[torch.Tensor] = None  # [numel] bytes: E4M3 copy written by the quantise-on-gather kernel
        self.grad: Optional[torch.Tensor] = None  # [numel] full-size gradient buffer
        self.grad_shard: Optional[torch.Tensor] = None  # [shard_numel] reduced gradient owned by this rank
        self.gather_work: Any = None
        self.reduce_work: Any = None
        self.grad_persistent = False  # gradient buffer lives in the symmetric arena for the whole run
        self.written: set = set()
        self.trainable = True
        self.expert = False  # expert-parallel bucket: this rank owns whole experts; never sharded or reduced across the EP group
        self.decay_mask_cache: Optional[torch.Tensor] = None

    def slot(self, name: str) -> Slot:
        for s in self.slots:
            if s.name == name:
                return s
        raise KeyError(name)


class SingleProcessComm:
    """Collectives for world size 1 (all are copies / no-ops)."""
    rank, world = 0, 1

    def all_gather(self, shard, full, async_op=False):
        if full.data_ptr() != shard.data_ptr():
            full.copy_(shard)
        return None

    def reduce_scatter(self, full, shard, async_op=False, average=True):
        if shard.data_ptr() != full.data_ptr():
            shard.copy_(full)
        return None

    def all_reduce(self, t, op="sum", async_op=False):
        return None

    def barrier(self):
        pass


class _HostGatherWork:
    """Completion handle of a host-sourced gather: makes the current stream wait for the copy (and the collective)."""

    def __init__(self, event, inner, keep):
        self.event, self.inner, self.keep = event, inner, keep

    def wait(self):
        if self.inner is not None:
            self.inner.wait()
        torch.cuda.current_stream().wait_event(self.event)
        self.keep = None


class ParamStore:
    def __init__(self, cm: CompiledModel, *, device, param_dtype=torch.float32, grad_dtype=None, master_dtype=None,
                 comm=None, zero_level: int = 0, keep_gathered: bool = True, frozen: Optional[Callable[[str], bool]] = None,
                 expert_parallel: int = 1, offload_master: bool = False, host_work_copy: bool = False,
                 owned: Optional[Callable[[Any], bool]] = None, resident_layers: int = 0, grad_mask=None, ep_comm=None, expert_dp_comm=None):
        self.cm = cm
        # with host-resident masters: the frozen weights of the first ``resident_layers`` layers stay in device memory instead,
        # so their per-traversal gather is NVLink / local traffic rather than PCIe (spend spare HBM on the layers used first)
        self.resident_layers = int(resident_layers)
        # pipeline stages: ``owned(entry)`` says whether this process holds the parameter at all; the others are never
        # allocated, initialised, loaded or stepped here
        self.owned = owned
        self.device = torch.device(device)
        self.param_dtype = param_dtype
        self.grad_dtype = grad_dtype or param_dtype
        self.master_dtype = master_dtype or param_dtype
        self.comm = comm or SingleProcessComm()
        self.world, self.rank = self.comm.world, self.comm.rank
        self.zero_level = zero_level if self.world > 1 else 0
        self.keep_gathered = keep_gathered
        self.frozen = frozen or (lambda name: False)
        self.grad_mask = grad_mask  # runtime.grad_mask.GradientMask: partial-update runs of a full model
        self.ep = max(1, int(expert_parallel))
        # expert-parallel x data-parallel mesh (parallel/mesh.py): the expert group is a sub-group of the world when dp > 1; expert
        # weights are gathered inside it and expert gradients are summed over the ranks that hold the same experts
        self.ep_comm = ep_comm if ep_comm is not None else self.comm
        self.expert_dp_comm = expert_dp_comm
        self.ep_rank = self.rank % self.ep
        self.expert_dp = expert_dp_comm.world if expert_dp_comm is not None else 1
        # Host residency: master shards live in pinned host memory and are streamed to the device per layer (H2D copy on a
        # side stream, then the usual gather).  ``host_work_copy`` keeps an extra pinned copy in the parameter dtype next to
        # masters of another dtype (fp32 masters updated by the CPU optimizer, bf16 copy streamed to the GPU).
        self.offload_master = bool(offload_master)
        self.host_work_copy = bool(host_work_copy) and self.offload_master
        self.host_work_double = host_work_copy == "double" and self.offload_master  # two copies: one being read, one being written by a stale update
        self.h2d_stream = torch.cuda.Stream(device=self.device) if (self.offload_master and self.device.type == "cuda") else None
        self.stage_slots: List[torch.Tensor] = []
        self._stage_rr = 0
        self.h2d_bytes = 0
        self.buckets: "OrderedDict[str, Bucket]" = OrderedDict()
        self.where: Dict[str, Tuple[Bucket, Slot]] = {}
        self.alias: Dict[str, str] = {}
        self.first_micro_step = True
        self.last_micro_step = True
        self.grads_enabled = True
        self.post_gather: Optional[Callable[[Bucket], None]] = None
        self.expert_placement: Dict[int, List[int]] = {}  # layer -> placed index of every global expert (expert parallelism with re-placement)
        self.fp8_gather = False  # quantise-on-gather (ZeRO-3 + FP8 recipe + peer-memory kernels)
        self.fp8_roles: Dict[str, str] = {}
        self._build()

    # ------------------------------------------------------------------ layout
    def _build(self) -> None:
        for e in self.cm.params:
            if self.owned is not None and not self.owned(e):
                continue
            if e.tied_to:
                self.alias[e.name] = e.tied_to
                continue
            shape = tuple(e.spec.shape)
            gname = e.group
            is_expert = self.ep > 1 and e.local.startswith("experts_")
            if is_expert:
                assert shape[0] % self.ep == 0, f"{e.name}: {shape[0]} experts do not divide over ep={self.ep}"
                shape = (shape[0] // self.ep,) + shape[1:]
                gname = e.group + ".experts"
            b = self.buckets.get(gname)
            if b is None:
                b = self.buckets[gname] = Bucket(gname, e.layer)
                b.expert = is_expert
            n = math.prod(shape)
            gm = self.grad_mask
            slot = Slot(e.name, b.numel, n, shape, e.spec.decay and (gm is None or gm.decays(e.name)), e,
                        trainable=not self.frozen(e.name) and (gm is None or gm.trainable(e.name)))
            b.slots.append(slot)
            b.numel += (n + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS
            self.where[e.name] = (b, slot)
        quantum = self.world * ALIGN_ELEMS
        for b in self.buckets.values():
            b.numel = (b.numel + quantum - 1) // quantum * quantum
            b.shard_numel = b.numel // self.world if (self.sharded and not b.expert) else b.numel
            b.trainable = any(s.trainable for s in b.slots)
        # Peer-addressable placement: when the communicator runs its own kernels over symmetric memory, master shards
        # and bucket-sized gradient buffers live in one arena so that peers can load them directly.
        self.arena = None
        self.fused_sumsq = None
        self.sumsq_valid = False
        self.micro_total = 1
        stream_dtype_ok = self.param_dtype == torch.bfloat16 and (self.master_dtype == torch.bfloat16 or self.host_work_copy)
        if hasattr(self.comm, "create_arena") and self.sharded and self.grad_dtype == torch.bfloat16 and \
                (stream_dtype_ok if self.offload_master else self.master_dtype == torch.bfloat16):
            need = 0
            max_shard = 0
            for b in self.buckets.values():
                if b.expert:
                    continue
                if self.offload_master and not self._resident(b):
                    max_shard = max(max_shard, b.shard_numel)
                else:
                    need += (b.shard_numel * 2 + 255) // 256 * 256 + 256
                if b.trainable:
                    need += (b.numel * 2 + 255) // 256 * 256 + 256
            need += 2 * ((max_shard * 2 + 255) // 256 * 256 + 256)
            self.arena = self.comm.create_arena(need)
            self.arena.tensor.zero_()
            self.fused_sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
            if self.offload_master:  # two peer-visible landing slots for the H2D copies that feed the gather kernel
                self.stage_slots = [self.arena.take(max_shard, torch.bfloat16) for _ in range(2)]
        pin = self.device.type == "cuda"
        for b in self.buckets.values():
            if b.expert:
                b.master = torch.zeros(b.numel, dtype=self.master_dtype, device=self.device)
                b.work = b.master if self.master_dtype == self.param_dtype else torch.zeros(b.numel, dtype=self.param_dtype, device=self.device)
                continue
            if self.offload_master and not self._resident(b):
                b.master = torch.zeros(b.shard_numel, dtype=self.master_dtype, pin_memory=pin)
                double = self.host_work_double  # one-step-stale optimizer: the update writes ``work_next`` while steps read ``work_host``
                b.work_host = torch.zeros(b.shard_numel, dtype=self.param_dtype, pin_memory=pin) if (
                    self.host_work_copy and (double or self.master_dtype != self.param_dtype)) else None
                b.work_next = torch.zeros(b.shard_numel, dtype=self.param_dtype, pin_memory=pin) if (double and b.trainable) else None
                if self.arena is not None and b.trainable:
                    b.grad = self.arena.take(b.numel, self.grad_dtype)
                    b.grad_persistent = True
                if self.zero_level < 3:
                    b.work = torch.zeros(b.numel, dtype=self.param_dtype, device=self.device)
                continue
            if self.arena is not None:
                b.master = self.arena.take(b.shard_numel, self.master_dtype)
                if b.trainable:
                    b.grad = self.arena.take(b.numel, self.grad_dtype)
                    b.grad_persistent = True
            else:
                b.master = torch.zeros(b.shard_numel, dtype=self.master_dtype, device=self.device)
            if not self.sharded and self.master_dtype == self.param_dtype:
                b.work = b.master
            elif self.zero_level < 3:
                b.work = torch.zeros(b.numel, dtype=self.param_dtype, device=self.device)

    def _resident(self, b: Bucket) -> bool:
        """Frozen layer buckets below ``resident_layers`` keep their master shard on the device although masters are offloaded."""
        return self.resident_layers > 0 and b.layer is not None and b.layer < self.resident_layers and not b.trainable and not b.expert \
            and self.master_dtype == self.param_dtype

    @property
    def sharded(self) -> bool:
        return self.zero_level >= 1

    def resolve(self, name: str) -> str:
        return self.alias.get(name, name)

    def shard_range(self, b: Bucket) -> Tuple[int, int]:
        if not self.sharded or b.expert:
            return 0, b.numel
        return self.rank * b.shard_numel, (self.rank + 1) * b.shard_numel

    # ------------------------------------------------------------------ init / import / export
    def init_weights(self, seed: int = 0, std: float = 0.02, zero_projections: bool = False) -> None:
        """Seeded N(0, std) init.  Every parameter (every expert of an expert parameter) has its own generator stream, so the
        values do not depend on the world size or the expert-parallel layout.  Large slots are generated on the GPU."""
        big = 1 << 24
        for bi, b in enumerate(self.buckets.values()):
            for si, s in enumerate(b.slots):
                base_seed = seed * 1000003 + (zlib.crc32(s.name.encode()) & 0xFFFFF) * 1009
                kind = s.entry.spec.init
                zero = kind == "zeros" or (zero_projections and s.entry.local in ("out_weight", "mlp_down_weight", "experts_down"))
                if b.expert:
                    El = s.shape[0]
                    per = s.numel // El
                    for j in range(El):
                        ge = self.ep_rank * El + j
                        t = self._gen(per, base_seed + 7 * ge, kind, zero, std, per >= big)
                        b.master[s.offset + j * per:s.offset + (j + 1) * per].copy_(t.to(self.master_dtype))
                    continue
                if s.entry.local.startswith("experts_") and len(s.shape) == 3:
                    # the same per-expert streams without expert parallelism, so a run does not depend on the expert-parallel degree
                    per = s.numel // s.shape[0]
                    flat = torch.cat([self._gen(per, base_seed + 7 * e, kind, zero, std, per >= big).cpu() for e in range(s.shape[0])])
                    self._write_master(b, s, flat)
                    continue
                self._write_master(b, s, self._gen(s.numel, base_seed, kind, zero, std, s.numel >= big))
        self.sync_work_from_master()

    def _gen(self, n: int, seed: int, kind: str, zero: bool, std: float, on_device: bool) -> torch.Tensor:
        dev = self.device if (on_device and self.device.type == "cuda") else torch.device("cpu")
        if kind == "ones":
            return torch.ones(n, device=dev)
        if zero:
            return torch.zeros(n, device=dev)
        gen = torch.Generator(device=dev).manual_seed(seed & 0x7FFFFFFFFFFF)
        return torch.empty(n, device=dev).normal_(0.0, std, generator=gen)

    def _write_master(self, b: Bucket, s: Slot, flat_cpu: torch.Tensor) -> None:
        lo, hi = self.shard_range(b)
        a, z = max(s.offset, lo), min(s.offset + s.numel, hi)
        if a < z:
            b.master[a - lo:z - lo].copy_(flat_cpu[a - s.offset:z - s.offset].to(self.master_dtype))

    def _expert_slice(self, s: Slot, tensor: torch.Tensor) -> torch.Tensor:
        El = s.shape[0]
        return tensor[self.ep_rank * El:(self.ep_rank + 1) * El]

    def holds(self, name: str) -> bool:
        return self.resolve(name) in self.where

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        name = self.resolve(name)
        if self.owned is not None and name not in self.where:
            return  # another pipeline stage's parameter
        b, s = self.where[name]
        if b.expert and tensor.shape[0] == s.shape[0] * self.ep:
            tensor = self._expert_slice(s, tensor)  # a full [E, ...] tensor: keep this rank's experts
        assert tuple(tensor.shape) == s.shape, f"{name}: expected {s.shape}, got {tuple(tensor.shape)}"
        self._write_master(b, s, tensor.reshape(-1))

    def full_tensor(self, name: str) -> torch.Tensor:
        """Gather one parameter in full on every rank (export / debug)."""
        name = self.resolve(name)
        b, s = self.where[name]
        if b.expert:
            flat = self._dequantized(b) if getattr(b, "qstate", None) is not None else b.master
            return self._gather_experts(flat[s.offset:s.offset + s.numel].reshape(s.shape), b.layer)
        if getattr(b, "qstate", None) is not None:
            return self._dequantized(b)[s.offset:s.offset + s.numel].reshape(s.shape)
        if not self.sharded:
            return self._master_on_device(b)[s.offset:s.offset + s.numel].reshape(s.shape)
        full = torch.empty(b.numel, dtype=self.master_dtype, device=self.device)
        self.comm.all_gather(self._master_on_device(b), full)
        return full[s.offset:s.offset + s.numel].reshape(s.shape)

    def _master_on_device(self, b: Bucket) -> torch.Tensor:
        return b.master if b.master.device == self.device else b.master.to(self.device)

    def _gather_experts(self, local: torch.Tensor, layer: Optional[int] = None) -> torch.Tensor:
        """[E/ep, ...] on every rank -> [E, ...] in global expert order (ranks hold E/ep slots each; which expert sits in
        which slot is the identity unless experts were re-placed for load balance)."""
        local = local.contiguous()
        full = torch.empty((self.ep * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        getattr(self.ep_comm, "base", self.ep_comm).all_gather(local.reshape(-1), full.reshape(-1))
        place = self.expert_placement.get(layer) if layer is not None else None
        if place is not None:
            full = full.index_select(0, torch.tensor(place, dtype=torch.long, device=full.device))
        return full

    def named_full_tensors(self) -> Iterable[Tuple[str, torch.Tensor]]:
        for b in self.buckets.values():
            if b.expert:
                flat = self._dequantized(b) if getattr(b, "qstate", None) is not None else b.master
                for s in b.slots:
                    yield s.name, self._gather_experts(flat[s.offset:s.offset + s.numel].reshape(s.shape), b.layer)
                continue
            if getattr(b, "qstate", None) is not None:
                full = self._dequantized(b)
            elif self.sharded:
                full = torch.empty(b.numel, dtype=self.master_dtype, device=self.device)
                self.comm.all_gather(self._master_on_device(b), full)
            else:
                full = self._master_on_device(b)
            for s in b.slots:
                yield s.name, full[s.offset:s.offset + s.numel].reshape(s.shape)

    def sync_work_from_master(self) -> None:
        """Refresh the gathered work weights after the masters changed (init, load, optimizer step)."""
        fence = getattr(self.comm, "fence", None)
        if fence is not None and self.sharded:
            fence()  # peers pull master shards directly: every rank must have finished writing its own first
        if self.fp8_gather:
            self.refresh_weight_scales()
        for b in self.buckets.values():
            if getattr(b, "qstate", None) is not None:   # frozen and quantised (dense layer buckets, managed expert buckets): rebuilt on use
                b.work = None
                continue
            if b.expert:
                if b.work is not b.master:
                    b.work.copy_(b.master)
                continue
            if getattr(b, "work_host", None) is not None and not getattr(b, "work_host_fresh", False):
                b.work_host.copy_(b.master)  # host-side conversion (init / load); the CPU optimizer writes it itself afterwards
            b.work_host_fresh = False
            if self.zero_level >= 3:
                b.work = None
                b.work_fp8 = None
                b.gather_work = None
                continue
            if b.work is b.master:
                continue
            self._gather_into(b, b.work)
            if self.post_gather is not None:
                self.post_gather(b)

    # ------------------------------------------------------------------ QLoRA: frozen buckets stored block-quantised
    def quantize_frozen(self, codec) -> int:
        """Replace the master copy of every frozen, non-expert layer bucket by its block-quantised form.  The bf16 work
        weights are then rebuilt per layer when the executor reaches it and dropped afterwards, so at any time only one or
        two layers exist in bf16.  Returns the number of bytes saved."""
        assert self.zero_level == 0 or self.world == 1, "quantised base weights are replicated: use zero_level 0 with QLoRA on more than one rank"
        self.codec = codec
        saved = 0
        for b in self.buckets.values():
            if b.trainable or b.expert or b.layer is None or getattr(b, "qstate", None) is not None:
                continue
            src = b.master if b.master.device == self.device else b.master.to(self.device)
            b.qstate = codec.quantize(src)
            before = b.master.numel() * b.master.element_size()
            after = sum(t.numel() * t.element_size() for t in b.qstate.values())
            saved += before - after
            b.master = torch.empty(0, dtype=self.master_dtype, device=self.device)
            b.work = None
        return saved

    def _dequantized(self, b: Bucket) -> torch.Tensor:
        mgr = getattr(b.qstate, "manager", None)      # expert buckets under the offload manager (runtime/expert_offload.py)
        if mgr is not None:
            return mgr.fetch(b.layer, self.param_dtype)
        return self.codec.dequantize(b.qstate, self.param_dtype)

    # ------------------------------------------------------------------ FP8 quantise-on-gather
    FP8_SLOT_ROLES = {"qkv_weight": "qkv", "out_weight": "out", "mlp_up_weight": "mlp_up", "mlp_down_weight": "mlp_down"}

    def enable_fp8_gather(self, wants: Callable[[Optional[int], str], bool]) -> bool:
        """Gather ZeRO-3 weights straight into FP8: the gather kernel pulls the peers' bf16 shards and writes E4M3 with the
        tensor's scale, so the gathered bf16 copy and the separate abs-max / quantise passes disappear.  ``wants(layer, role)``
        says which projections the recipe runs in FP8.  Needs the peer-memory communicator and an arena."""
        if self.zero_level < 3 or self.arena is None or self.param_dtype != torch.bfloat16 or self.offload_master:
            return False
        self.q_index: Dict[str, int] = {}
        for b in self.buckets.values():
            if b.layer is None or b.expert:
                continue
            for sl in b.slots:
                role = self.FP8_SLOT_ROLES.get(sl.entry.local)
                if role and wants(b.layer, role):
                    self.q_index[sl.name] = len(self.q_index)
        if not self.q_index or len(self.q_index) > 1024:
            return False
        n = len(self.q_index)
        self.w_amax = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.w_scale = torch.ones(n, dtype=torch.float32, device=self.device)
        self.w_scale_inv = torch.ones(n, dtype=torch.float32, device=self.device)
        self.fp8_gather = True
        # Quantise-then-gather: every rank keeps an E4M3 copy of its own master shard in a second peer-visible arena, refreshed
        # once per optimizer step, and the gather pulls those bytes: one byte per weight crosses NVLink instead of two, and the
        # conversion work is done once by the owner instead of by every rank on arrival.
        self.fp8_arena = None
        alloc = getattr(self.comm, "_alloc_symmetric", None)
        if alloc is not None and self.sharded and self.master_dtype == torch.bfloat16 and os.environ.get("SUROGATE_FP8_SHARDS", FP8_SHARDS_DEFAULT) != "0":
            qb = [b for b in self.buckets.values() if b.layer is not None and not b.expert and any(sl.name in self.q_index for sl in b.slots)]
            total = sum((b.shard_numel + 255) // 256 * 256 for b in qb) + 4096
            try:
                self.fp8_arena = alloc(total)
                for b in qb:
                    b.master_fp8 = self.fp8_arena.take(b.shard_numel, torch.uint8)
            except Exception:  # noqa: BLE001 -- no room for a second arena: quantise on arrival as before
                self.fp8_arena = None
                for b in qb:
                    b.master_fp8 = None
        return True

    def refresh_weight_scales(self) -> None:
        """Per-tensor scales of the FP8 weights from the current masters: shard-local abs-max, one small max all-reduce."""
        from ..ops import ext

        e = ext()
        self.w_amax.zero_()
        for b in self.buckets.values():
            lo, hi = self.shard_range(b)
            for sl in b.slots:
                i = self.q_index.get(sl.name)
                if i is None:
                    continue
                a, z = max(sl.offset, lo), min(sl.offset + sl.numel, hi)
                if a < z:
                    e.amax(b.master[a - lo:z - lo], self.w_amax[i:i + 1])
        self.comm.all_reduce(self.w_amax, "max")
        torch.where(self.w_amax > 0, 448.0 / self.w_amax, torch.ones_like(self.w_amax), out=self.w_scale)
        torch.reciprocal(self.w_scale, out=self.w_scale_inv)
        if getattr(self, "fp8_arena", None) is not None:
            for b in self.buckets.values():
                dst = getattr(b, "master_fp8", None)
                if dst is None:
                    continue
                lo, hi = self.shard_range(b)
                for sl in b.slots:
                    i = self.q_index.get(sl.name)
                    if i is None:
                        continue
                    a, z = max(sl.offset, lo), min((sl.offset + sl.numel + 15) // 16 * 16, hi)
                    if a < z:
                        e.quantize_fp8(b.master[a - lo:z - lo], self.w_scale[i:i + 1], None, False, None, dst[a - lo:z - lo])
            fence = getattr(self.comm, "fence", None)
            if fence is not None:
                fence()      # the peers pull these bytes: every rank's copy must be complete before the first gather of the next step

    def get_fp8(self, name: str):
        """(E4M3 weight view, de-scale) of a parameter gathered in FP8, or None."""
        if not self.fp8_gather:
            return None
        name = self.resolve(name)
        i = self.q_index.get(name)
        if i is None:
            return None
        b, sl = self.where[name]
        if b.work_fp8 is None or b.gather_work is not None:
            self._ensure_gathered(b)
        return b.work_fp8[sl.offset:sl.offset + sl.numel].view(sl.shape).view(torch.float8_e4m3fn), self.w_scale_inv[i:i + 1]

    def _gather_fp8(self, b: Bucket):
        """One fused pull per parameter: FP8 for the quantised projections, bf16 for the rest (norm weights ...)."""
        b.work = torch.empty(b.numel, dtype=self.param_dtype, device=self.device)
        b.work_fp8 = torch.empty(b.numel, dtype=torch.uint8, device=self.device)
        works = []
        for sl in b.slots:
            end = (sl.offset + sl.numel + 7) // 8 * 8
            i = self.q_index.get(sl.name)
            if i is not None and getattr(b, "master_fp8", None) is not None:
                w = self.comm.all_gather_bytes(b.master_fp8, b.work_fp8, self.fp8_arena, (sl.offset, (sl.offset + sl.numel + 15) // 16 * 16), async_op=True)
            elif i is not None:
                w = self.comm.all_gather(b.master, None, async_op=True, out_fp8=b.work_fp8, scale=self.w_scale[i:i + 1], segment=(sl.offset, end))
            else:
                w = self.comm.all_gather(b.master, b.work, async_op=True, segment=(sl.offset, end))
            works.append(w)
        return works[-1] if works else None   # same communication stream: the last event covers all of them

    def host_source(self, b: Bucket) -> torch.Tensor:
        """The pinned host tensor streamed to the GPU for this bucket (in the parameter dtype when one exists)."""
        wh = getattr(b, "work_host", None)
        return wh if wh is not None else b.master

    def _gather_from_host(self, b: Bucket, full: torch.Tensor, async_op: bool):
        """Pinned host shard -> device -> (all-gather) -> ``full``, entirely on side streams."""
        src = self.host_source(b)
        self.h2d_bytes += src.numel() * src.element_size()
        if self.sharded and self.stage_slots and src.dtype == torch.bfloat16 and full.dtype == torch.bfloat16 and hasattr(self.comm, "all_gather_from_host"):
            k = self._stage_rr
            self._stage_rr ^= 1
            return self.comm.all_gather_from_host(src, self.stage_slots[k][:src.numel()], full, async_op=async_op)
        cur = torch.cuda.current_stream(self.device)
        hs = self.h2d_stream
        hs.wait_stream(cur)  # blocks handed out by the allocator may still be in use by kernels queued on the compute stream
        with torch.cuda.stream(hs):
            stage = torch.empty(src.numel(), dtype=src.dtype, device=self.device)
            stage.copy_(src, non_blocking=True)
            dev = stage if stage.dtype == full.dtype else stage.to(full.dtype)
            inner = None
            if not self.sharded:
                full.copy_(dev)
            else:
                inner = self.comm.all_gather(dev, full, async_op=True)
            ev = torch.cuda.Event()
            ev.record(hs)
            for t in (stage, dev, full):
                t.record_stream(hs)
        h = _HostGatherWork(ev, inner, (stage, dev))
        if not async_op:
            h.wait()
            return None
        return h

    def _gather_into(self, b: Bucket, full: torch.Tensor, async_op: bool = False):
        if b.master.device.type == "cpu" and self.device.type == "cuda":
            return self._gather_from_host(b, full, async_op)
        base = self.host_source(b) if b.master.device.type == "cpu" else b.master  # host masters: the published copy (a stale update may be writing the masters)
        src = base if base.dtype == full.dtype else base.to(full.dtype)
        if not self.sharded:
            full.copy_(src)
            return None
        return self.comm.all_gather(src, full, async_op=async_op)

    # ------------------------------------------------------------------ executor hooks
    def _ensure_gathered(self, b: Bucket, prefetch_only: bool = False) -> None:
        if b.work is None and getattr(b, "qstate", None) is not None:
            b.work = self._dequantized(b)
            b._needs_post = True
        if b.work is None:
            if self.fp8_gather and b.layer is not None and not b.expert:
                b.gather_work = self._gather_fp8(b)
            else:
                b.work = torch.empty(b.numel, dtype=self.param_dtype, device=self.device)
                b.gather_work = self._gather_into(b, b.work, async_op=True)
            b._needs_post = True
        if not prefetch_only:
            if b.gather_work is not None:
                b.gather_work.wait()
                b.gather_work = None
            if getattr(b, "_needs_post", False):
                b._needs_post = False
                if self.post_gather is not None:
                    self.post_gather(b)

    def _release(self, b: Bucket) -> None:
        if getattr(b, "qstate", None) is not None:
            b.work = None
            return
        if self.zero_level >= 3 and not b.expert:
            b.work = None
            b.work_fp8 = None

    def _layer_bucket(self, L: int) -> Optional[Bucket]:
        return self.buckets.get(f"layer{L}")

    def layer_start(self, L: int, phase: str) -> None:
        mgr = getattr(self, "expert_offload", None)
        if mgr is not None:       # quantised experts stream one MoE layer ahead of their use
            mgr.prefetch(L)
            nxt_moe = mgr.neighbours(L, phase)
            if nxt_moe is not None:
                mgr.prefetch(nxt_moe)
        if self.zero_level < 3:
            b = self._layer_bucket(L)
            if b is not None and getattr(b, "qstate", None) is not None:
                self._ensure_gathered(b)
            return
        b = self._layer_bucket(L)
        self._ensure_gathered(b)
        nxt = L + 1 if phase == "fwd" else L - 1
        nb = self._layer_bucket(nxt)
        if nb is not None:
            self._ensure_gathered(nb, prefetch_only=True)

    def layer_end(self, L: int, phase: str) -> None:
        b = self._layer_bucket(L)
        if b is None:
            return
        eb = self.buckets.get(f"layer{L}.experts")
        if phase == "bwd":
            self._reduce_bucket(b)
            self._release(b)
            if eb is not None:
                self._reduce_bucket(eb)
        elif not self.keep_gathered or getattr(b, "qstate", None) is not None:
            self._release(b)
        if eb is not None and getattr(eb, "qstate", None) is not None:
            eb.work = None          # the dequantised experts of this layer are rebuilt when it is next reached

    def group_start(self, group: str, phase: str) -> None:
        pass

    def group_end(self, group: str, phase: str) -> None:
        """Called after the whole backward: reduce the non-layer buckets (embedding, final norm, LM head)."""
        for b in self.buckets.values():
            if b.layer is None:
                self._reduce_bucket(b)
                if self.zero_level >= 3:
                    self._release(b)

    def get(self, name: str) -> torch.Tensor:
        name = self.resolve(name)
        b, s = self.where[name]
        if b.work is None or b.gather_work is not None or getattr(b, "_needs_post", False):
            self._ensure_gathered(b)
        return b.work[s.offset:s.offset + s.numel].view(s.shape)

    # ------------------------------------------------------------------ gradients
    def begin_step(self) -> None:
        for b in self.buckets.values():
            b.written.clear()
        self.first_micro_step = True
        if self.fused_sumsq is not None:
            self.fused_sumsq.zero_()
            self.sumsq_valid = True

    def begin_micro_step(self, index: int, total: int) -> None:
        self.first_micro_step = index == 0
        self.last_micro_step = index == total - 1
        self.micro_total = total
        if self.zero_level >= 2:
            for b in self.buckets.values():
                b.written.clear()

    def grad_target(self, name: str):
        if not self.grads_enabled:
            return None, False
        name = self.resolve(name)
        b, s = self.where[name]
        if not s.trainable:
            return None, False
        if b.grad is None:
            b.grad = torch.zeros(b.numel, dtype=self.grad_dtype, device=self.device)
        acc = name in b.written
        b.written.add(name)
        return b.grad[s.offset:s.offset + s.numel].view(s.shape), acc

    def _reduce_bucket(self, b: Bucket, zero_unwritten: bool = True) -> None:
        """Start the (async) gradient reduction of one bucket; called as soon as its backward is complete.
        With ``defer_reduce`` (forward + backward captured in a CUDA graph: the collectives stay outside the graph) only the
        zero-fill of parameters without a gradient happens here; ``reduce_deferred`` starts the reductions afterwards."""
        if b.grad is None or not b.trainable:
            return
        for s in (b.slots if zero_unwritten else ()):  # parameters that received no gradient this micro-step contribute zeros
            if s.trainable and s.name not in b.written and (self.zero_level >= 2 or b.grad_persistent):
                b.grad[s.offset:s.offset + s.numel].zero_()
        if self.grad_mask is not None and zero_unwritten:  # before the reduction: the zeroed half costs no precision in the sum
            for s in b.slots:
                if s.trainable and self.grad_mask.has_partial(s.name):
                    self.grad_mask.apply_partial(s.name, b.grad[s.offset:s.offset + s.numel].view(s.shape))
        if getattr(self, "defer_reduce", False):
            return
        if self.world == 1 or b.expert:
            b.grad_shard = b.grad  # whole experts live on this rank: nothing to reduce inside the expert group
            if b.expert and self.expert_dp > 1 and self.last_micro_step:
                # the replicas of the expert group saw different tokens: sum their expert gradients (and over nothing else)
                b.reduce_work = self.expert_dp_comm.all_reduce(b.grad, op="sum", async_op=True)
            return
        if self.zero_level == 0:
            self.sumsq_valid = False
            if self.last_micro_step:
                b.reduce_work = self.comm.all_reduce(b.grad, op="sum", async_op=True)  # loss is normalised by the global token count
                b.grad_shard = b.grad
            return
        if self.zero_level == 1 or self.micro_total == 1:
            # one reduction per bucket per step: asynchronous, overlapped with the rest of backward, and (with the
            # peer-memory kernels) fused with the sum of squares for the gradient norm
            if self.last_micro_step:
                b.grad_shard = torch.empty(b.shard_numel, dtype=self.grad_dtype, device=self.device)
                b.reduce_work = self._reduce_scatter(b.grad, b.grad_shard)
                if not b.grad_persistent and self.zero_level >= 2:
                    b.grad = None
            return
        # level 2/3 with gradient accumulation: reduce-scatter every micro-step into an fp32 accumulator
        self.sumsq_valid = False
        tmp = torch.empty(b.shard_numel, dtype=self.grad_dtype, device=self.device)
        w = self.comm.reduce_scatter(b.grad, tmp, async_op=True)
        if w is not None:
            w.wait()
        if b.grad_shard is None or self.first_micro_step:
            b.grad_shard = tmp.float()
        else:
            b.grad_shard = b.grad_shard + tmp.float()
        if not b.grad_persistent:
            b.grad = None

    def _reduce_scatter(self, full: torch.Tensor, shard: torch.Tensor):
        if self.fused_sumsq is not None and self.arena.offset_of(full) is not None:
            return self.comm.reduce_scatter(full, shard, async_op=True, sumsq_out=self.fused_sumsq)
        self.sumsq_valid = False
        return self.comm.reduce_scatter(full, shard, async_op=True)

    def reduce_deferred(self) -> None:
        """Reductions of every bucket after a graph-replayed backward (the write bookkeeping of a replay lives in the graph, so
        nothing is zero-filled here)."""
        self.defer_reduce = False
        for b in self.buckets.values():
            self._reduce_bucket(b, zero_unwritten=False)

    def finish_reduce(self) -> None:
        for b in self.buckets.values():
            if b.reduce_work is not None:
                b.reduce_work.wait()
                b.reduce_work = None
            if b.grad_shard is None and b.grad is not None and b.trainable:
                b.grad_shard = b.grad

    def trainable_buckets(self) -> List[Bucket]:
        return [b for b in self.buckets.values() if b.trainable]

    def decay_mask(self, b: Bucket) -> torch.Tensor:
        """Per-element 0/1 weight-decay mask of this rank's shard (1 for matrices, 0 for norms/biases/padding)."""
        if b.decay_mask_cache is None:
            lo, hi = self.shard_range(b)
            m = torch.zeros(hi - lo, dtype=torch.uint8, device=self.device)
            for s in b.slots:
                if s.decay and s.trainable:
                    a, z = max(s.offset, lo), min(s.offset + s.numel, hi)
                    if a < z:
                        m[a - lo:z - lo] = 1
            b.decay_mask_cache = m
        return b.decay_mask_cache

    def decay_mask_blocks(self, b: Bucket) -> torch.Tensor:
        """The same mask at one byte per 128 elements (slots start on 128-element boundaries and shards are multiples of 128,
        so nothing is lost); what the optimizer kernels read."""
        m = getattr(b, "decay_blocks_cache", None)
        if m is None:
            full = self.decay_mask(b)
            assert full.numel() % ALIGN_ELEMS == 0
            m = b.decay_blocks_cache = full.view(-1, ALIGN_ELEMS).amax(1).contiguous()
        return m

    def grad_of(self, name: str) -> Optional[torch.Tensor]:
        """Full (reduced) gradient of one parameter — debugging / tests; gathers when sharded."""
        name = self.resolve(name)
        b, s = self.where[name]
        g = b.grad_shard if b.grad_shard is not None else b.grad
        if g is None:
            return None
        if b.expert:
            return self._gather_experts(g[s.offset:s.offset + s.numel].view(s.shape), b.layer)
        if g.numel() != b.numel:
            full = torch.empty(b.numel, dtype=g.dtype, device=self.device)
            self.comm.all_gather(g.contiguous(), full)
            g = full
        return g[s.offset:s.offset + s.numel].view(s.shape)

    def release_grads(self) -> None:
        for b in self.buckets.values():
            if b.expert:
                b.grad_shard = None
                continue
            if self.zero_level >= 1:
                b.grad_shard = None
            if self.zero_level >= 2 and not b.grad_persistent:
                b.grad = None

    def memory_breakdown(self) -> Dict[str, int]:
        out = {"master": 0, "work": 0, "grad": 0, "host_master": 0}
        for b in self.buckets.values():
            out["master" if b.master.device.type != "cpu" or self.device.type == "cpu" else "host_master"] += b.master.numel() * b.master.element_size()
            if b.work is not None and b.work is not b.master:
                out["work"] += b.work.numel() * b.work.element_size()
            if b.grad is not None:
                out["grad"] += b.grad.numel() * b.grad.element_size()
        return out

"""Host-resident training state: streamed optimizer step and the CPU optimizer path.

Three arrangements, all using pinned host memory and ``cudaMemcpyAsync`` on side streams:

* ``offload_optimizer`` — optimizer moments live on the host; per bucket they are copied in on one stream, updated by the
  ordinary GPU kernel, and copied back on another stream, so the H2D of bucket *i+1* overlaps the D2H of bucket *i*
  (PCIe is full duplex) and both overlap the update kernels.
* ``offload_master`` — master weight shards live on the host too and take the same round trip (frozen masters, as in
  LoRA, are only ever read: the per-layer gather streams them in, nothing is written back).
* ``cpu_training`` — fp32 masters and fp32 AdamW moments stay on the host, reduced gradient shards are copied out
  per bucket and the update runs on the CPU (native OpenMP kernel), which also writes the bf16 copy that the next
  step's weight streaming reads.

Parity: csrc/src/runtime/optimizers/cpu_adamw.cpp, adamw_8bit_optimizer.cpp:702-825 (CPU path), dsl_grad_store.cpp:727-1010
(per-layer D2H of gradients), docs/guides/offloading.md.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch


class StreamedOptimizerStep:
    """Runs ``optimizer.step_bucket`` over buckets whose master and/or moments are host-resident."""

    def __init__(self, store, optimizer, device):
        self.store, self.opt, self.device = store, optimizer, device
        self.on_gpu = device.type == "cuda"
        self.in_stream = torch.cuda.Stream(device=device) if self.on_gpu else None
        self.out_stream = torch.cuda.Stream(device=device) if self.on_gpu else None
        self.bytes_in = 0
        self.bytes_out = 0

    def _to_device(self, t: torch.Tensor) -> torch.Tensor:
        if t.device == self.device or not self.on_gpu:
            return t
        d = torch.empty(t.shape, dtype=t.dtype, device=self.device)
        d.copy_(t, non_blocking=True)
        self.bytes_in += t.numel() * t.element_size()
        return d

    def _stage_in(self, b):
        """Device copies of everything the update kernel touches for bucket ``b`` (on the H2D stream)."""
        main = torch.cuda.current_stream(self.device) if self.on_gpu else None
        host_state = self.opt.state_tensors(b)
        if not self.on_gpu:
            return b.master, host_state, None
        self.in_stream.wait_stream(main)
        with torch.cuda.stream(self.in_stream):
            master = self._to_device(b.master)
            state = {k: self._to_device(v) for k, v in host_state.items()}
            ev = torch.cuda.Event()
            ev.record(self.in_stream)
            for t in [master] + list(state.values()):
                t.record_stream(main)
                t.record_stream(self.out_stream)
        return master, state, ev

    def run(self, buckets: List, hp: torch.Tensor, hp_host) -> None:
        todo = [b for b in buckets if b.grad_shard is not None]
        if not todo:
            return
        main = torch.cuda.current_stream(self.device) if self.on_gpu else None
        staged = self._stage_in(todo[0])
        for i, b in enumerate(todo):
            master_dev, state_dev, ev = staged
            if ev is not None:
                main.wait_event(ev)
            host_master, host_state = b.master, self.opt.state.get(b.name)
            b.master, self.opt.state[b.name] = master_dev, state_dev
            try:
                self.opt.step_bucket(b, b.grad_shard, hp, hp_host)
            finally:
                b.master, self.opt.state[b.name] = host_master, host_state
            if self.on_gpu:
                done = torch.cuda.Event()
                done.record(main)
            if i + 1 < len(todo):
                staged = self._stage_in(todo[i + 1])  # queued behind this bucket's kernel; overlaps the write-back below
            if not self.on_gpu:
                continue
            self.out_stream.wait_event(done)
            with torch.cuda.stream(self.out_stream):
                if host_master.device.type == "cpu":
                    host_master.copy_(master_dev, non_blocking=True)
                    self.bytes_out += host_master.numel() * host_master.element_size()
                for k, v in host_state.items():
                    if v.device.type == "cpu":
                        v.copy_(state_dev[k], non_blocking=True)
                        self.bytes_out += v.numel() * v.element_size()
        if self.on_gpu:
            main.wait_stream(self.out_stream)  # the next step's weight streaming must see the written-back masters
            self.out_stream.synchronize()


class CpuAdamW:
    """fp32 AdamW on host-resident masters (native OpenMP kernel; PyTorch CPU ops when the host runtime is not built)."""
    state_bytes_per_param = 8

    def __init__(self, cfg, store, stale: Optional[str] = None):
        """``stale``: None = the update runs inside ``step_all``; "overlap" = the update of step N runs on a native worker thread
        while step N+1 computes with the weights of update N-1 (one-step stale; csrc/src/runtime/optimizers/async_optimizer.h);
        "inline" = the same staleness and bookkeeping (double-buffered gradients and work copies) with the update run in place
        instead of on the worker: the overlapped run must reproduce its trajectory bit for bit (the determinism check)."""
        self.cfg, self.store = cfg, store
        self.state: Dict[str, Dict[str, torch.Tensor]] = {}
        self.grad_host: Dict[str, torch.Tensor] = {}
        self.stale = stale
        self.worker = None
        self._pending: list = []          # buckets whose ``work_next`` holds the weights of the update in flight
        self._grad_sets = ({}, {})        # the worker reads one set while the next backward fills the other
        self._parity = 0
        self.d2h_stream = torch.cuda.Stream(device=store.device) if store.device.type == "cuda" else None
        self.bytes_out = 0
        try:
            from ..ops import host

            self.host = host()
        except Exception:  # noqa: BLE001
            self.host = None

    def _state(self, b):
        st = self.state.get(b.name)
        if st is None:
            n = b.master.numel()
            st = self.state[b.name] = {"m": torch.zeros(n, dtype=torch.float32), "v": torch.zeros(n, dtype=torch.float32)}
        return st

    state_tensors = _state

    def start_grad_copy(self, b) -> None:
        """Queue the D2H copy of the bucket's reduced gradient shard (called as soon as the shard is final)."""
        g = b.grad_shard
        if g is None:
            return
        if g.device.type == "cpu":
            self.grad_host[b.name] = g
            return
        pool = self._grad_sets[self._parity] if self.stale else self.grad_host
        h = pool.get(b.name)
        if h is None or h.shape != g.shape or h.dtype != g.dtype:
            h = pool[b.name] = torch.empty(g.shape, dtype=g.dtype, pin_memory=True)
        self.grad_host[b.name] = h
        self.d2h_stream.wait_stream(torch.cuda.current_stream(self.store.device))
        with torch.cuda.stream(self.d2h_stream):
            h.copy_(g, non_blocking=True)
            g.record_stream(self.d2h_stream)
        self.bytes_out += g.numel() * g.element_size()

    # ------------------------------------------------------------------ one-step-stale updates
    def close(self) -> None:
        """Wait for the update in flight, publish its weights and stop the worker.  Safe to call more than once."""
        if self.worker is not None:
            try:
                self.flush()
            finally:
                self.worker = None

    def __del__(self):
        try:
            w = self.worker
            if w is not None:
                w.drain()
        except Exception:  # noqa: BLE001  (interpreter shutdown: nothing to report to)
            pass

    def flush(self) -> None:
        """Wait for the update in flight and publish its weights (swap the work copies).  Called before the next update is
        queued and before anything reads masters or optimizer state (checkpoint, export, evaluation)."""
        if self.worker is not None:
            self.worker.drain()
        for b in self._pending:
            b.work_host, b.work_next = b.work_next, b.work_host
        self._pending = []

    def _submit_stale(self, buckets, lr: float, clip: float, step: int) -> None:
        if self.host is None:
            raise RuntimeError("the one-step-stale optimizer needs the native host runtime (surogate_b200.ops.build_host)")
        if self.worker is None:
            import atexit
            import weakref

            self.worker = self.host.AsyncAdamW(self.stale == "overlap")
            ref = weakref.ref(self)

            def _join_worker_before_shutdown():  # the worker thread is joined while the interpreter and the OpenMP runtime are still whole
                me = ref()
                if me is not None and me.worker is not None:
                    me.worker.drain()
                    me.worker = None

            atexit.register(_join_worker_before_shutdown)
        self.flush()
        c = self.cfg
        jobs, keep = [], []
        for b in buckets:
            g = self.grad_host.get(b.name)
            if g is None:
                continue
            if g.device.type != "cpu" or not g.is_contiguous():
                raise RuntimeError("stale updates read gradients from host memory")
            if g.data_ptr() == getattr(b.grad_shard, "data_ptr", lambda: 0)():  # CPU device: the gradient buffer itself is overwritten by the next backward
                h = self._grad_sets[self._parity].get(b.name)
                if h is None or h.shape != g.shape or h.dtype != g.dtype:
                    h = self._grad_sets[self._parity][b.name] = torch.empty_like(g)
                h.copy_(g)
                g = h
            st = self._state(b)
            assert b.master.dtype == torch.float32 and b.master.device.type == "cpu", "the CPU optimizer needs fp32 host masters"
            assert b.work_next is not None and b.work_host is not None, "stale updates need the double-buffered host work copy"
            mask = getattr(b, "decay_mask_host", None)
            if mask is None:
                mask = b.decay_mask_host = self.store.decay_mask(b).to("cpu").contiguous()
            if g.dtype not in (torch.float32, torch.bfloat16) or b.work_next.dtype not in (torch.float32, torch.bfloat16):
                raise RuntimeError(f"stale updates support fp32 / bf16 gradients and weights, got {g.dtype} / {b.work_next.dtype}")
            keep.extend((g, b.master, st["m"], st["v"], b.work_next, mask))
            jobs.append((b.master.data_ptr(), st["m"].data_ptr(), st["v"].data_ptr(), g.data_ptr(), g.dtype == torch.bfloat16, b.work_next.data_ptr(),
                         b.work_next.dtype == torch.bfloat16, b.master.numel(), mask.data_ptr()))
            self._pending.append(b)
            b.work_host_fresh = True  # the published copy stays what steps read; nothing may copy from the masters while they are being written
        # the worker owns a reference to every buffer of the update until it has completed (and waits for it in its own destructor),
        # so an optimizer or trainer dropped with an update in flight frees nothing that is still being written
        self.worker.submit(jobs, lr, c.beta1, c.beta2, c.eps, c.weight_decay, clip, step, keep)
        self.grad_host.clear()
        self._parity ^= 1

    def step_all(self, buckets, lr: float, clip: float, step: int) -> None:
        for b in buckets:
            if b.name not in self.grad_host:
                self.start_grad_copy(b)
        if self.d2h_stream is not None:
            self.d2h_stream.synchronize()
        c = self.cfg
        if self.stale:
            self._submit_stale(buckets, lr, clip, step)
            return
        for b in buckets:
            g = self.grad_host.get(b.name)
            if g is None:
                continue
            st = self._state(b)
            n = b.master.numel()
            assert b.master.dtype == torch.float32 and b.master.device.type == "cpu", "the CPU optimizer needs fp32 host masters"
            mask = getattr(b, "decay_mask_host", None)
            if mask is None:
                mask = b.decay_mask_host = self.store.decay_mask(b).to("cpu").contiguous()
            wh = getattr(b, "work_host", None)
            if self.host is not None and g.dtype in (torch.float32, torch.bfloat16):
                self.host.cpu_adamw_step(b.master.data_ptr(), st["m"].data_ptr(), st["v"].data_ptr(), g.data_ptr(), g.dtype == torch.bfloat16,
                                         wh.data_ptr() if wh is not None else 0, n, lr, c.beta1, c.beta2, c.eps, c.weight_decay, clip, step,
                                         mask.data_ptr())
            else:  # no native runtime (or an unusual gradient dtype)
                if clip == 0.0:  # skipped update (non-finite gradient norm)
                    if wh is not None:
                        wh.copy_(b.master)
                        b.work_host_fresh = True
                    continue
                gf = g.float() * clip
                st["m"].mul_(c.beta1).add_(gf, alpha=1 - c.beta1)
                st["v"].mul_(c.beta2).addcmul_(gf, gf, value=1 - c.beta2)
                bc1, bc2 = 1 - c.beta1 ** step, 1 - c.beta2 ** step
                p = b.master
                p.mul_(1 - lr * c.weight_decay * mask.float())
                p.addcdiv_(st["m"], (st["v"] / bc2).sqrt_().add_(c.eps), value=-lr / bc1)
                if wh is not None:
                    wh.copy_(p)
            if wh is not None:
                b.work_host_fresh = True
        self.grad_host.clear()

"""Quantised expert weights of frozen MoE layers, parked in pinned host memory and streamed one layer ahead (QLoRA on MoE models).

A Qwen3-30B-A3B style model is 90 % expert weights.  Under QLoRA they are frozen, so they can be held block-quantised (4.5 bits
per weight with NF4 + double quantisation) and, where even that does not fit next to activations, in pinned host memory.  The
manager owns, per MoE layer, the quantised state of the layer's expert bucket and moves it through three places:

    host (pinned)  --cudaMemcpyAsync on a side stream, one layer ahead-->  device staging slot (2 slots, ping-pong)
    device staging slot  --dequantise kernels-->  bf16 work buffer of the bucket (dropped when the layer is done)

``prefetch(L)`` is issued when layer L-1 (forward) or L+1 (backward) starts, ``fetch(L)`` waits for the copy and dequantises.
With ``offload=False`` the quantised state stays in device memory and only the dequantise step remains.

Parity: csrc/src/runtime/qlora/offload_manager.cpp (expert offload with prefetch), generic_weight_manager.cpp.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch


class ExpertOffloadManager:
    def __init__(self, store, codec, offload: bool = True, slots: int = 2):
        self.store, self.codec, self.offload = store, codec, offload
        self.device = store.device
        self.cuda = self.device.type == "cuda"
        self.host: Dict[int, Dict[str, torch.Tensor]] = {}        # layer -> quantised state (pinned host, or device when not offloading)
        self.staged: Dict[int, Dict[str, Any]] = {}               # layer -> {"state": device tensors, "event": copy done}
        self.slots = max(2, slots)
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.bytes_saved = 0
        self.h2d_bytes = 0
        self.layers: List[int] = []

    # ------------------------------------------------------------------ set-up
    def attach(self) -> int:
        """Quantise every frozen expert bucket, free its master copy.  Returns the bytes saved on the device."""
        for b in self.store.buckets.values():
            if not b.expert or b.trainable or b.layer is None or getattr(b, "qstate", None) is not None:
                continue
            src = b.master if b.master.device == self.device else b.master.to(self.device)
            st = self.codec.quantize(src)
            before = b.master.numel() * b.master.element_size()
            after = sum(t.numel() * t.element_size() for t in st.values())
            if self.offload and self.cuda:
                st = {k: (v.to("cpu").pin_memory() if v.device.type == "cuda" else v.pin_memory()) for k, v in st.items()}
                after = 0
            self.host[b.layer] = st
            self.bytes_saved += before - after
            b.master = torch.empty(0, dtype=self.store.master_dtype, device=self.device)
            b.work = None
            b.qstate = _ManagedState(self, b.layer)       # ParamStore._dequantized asks the codec; the proxy routes it here
            self.layers.append(b.layer)
        self.layers.sort()
        return self.bytes_saved

    # ------------------------------------------------------------------ streaming
    def prefetch(self, layer: int) -> None:
        if layer not in self.host or layer in self.staged:
            return
        st = self.host[layer]
        if not (self.offload and self.cuda):
            self.staged[layer] = {"state": st, "event": None}
            return
        while len(self.staged) >= self.slots:      # drop the oldest staged layer that is not the one being fetched
            self.staged.pop(next(iter(self.staged)))
        self.stream.wait_stream(torch.cuda.current_stream(self.device))   # the slot's previous user has finished with it
        with torch.cuda.stream(self.stream):
            dev = {k: v.to(self.device, non_blocking=True) for k, v in st.items()}
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.h2d_bytes += sum(v.numel() * v.element_size() for v in st.values())
        self.staged[layer] = {"state": dev, "event": ev}

    def fetch(self, layer: int, dtype: torch.dtype) -> torch.Tensor:
        self.prefetch(layer)
        item = self.staged.pop(layer)
        if item["event"] is not None:
            torch.cuda.current_stream(self.device).wait_event(item["event"])
            for v in item["state"].values():
                v.record_stream(torch.cuda.current_stream(self.device))
        return self.codec.dequantize(item["state"], dtype)

    def neighbours(self, layer: int, phase: str) -> Optional[int]:
        """The MoE layer that will be needed after ``layer`` in this phase."""
        later = [l for l in self.layers if l > layer] if phase == "fwd" else [l for l in reversed(self.layers) if l < layer]
        return later[0] if later else None

    def stats(self) -> Dict[str, float]:
        return {"expert_offload/layers": float(len(self.layers)), "expert_offload/device_bytes_saved": float(self.bytes_saved),
                "expert_offload/h2d_bytes": float(self.h2d_bytes), "expert_offload/offloaded": float(self.offload and self.cuda)}


class _ManagedState(dict):
    """Stands where a bucket's quantised state would be; ``ParamStore._dequantized`` recognises it and asks the manager."""

    def __init__(self, manager: ExpertOffloadManager, layer: int):
        super().__init__()
        self.manager, self.layer = manager, layer

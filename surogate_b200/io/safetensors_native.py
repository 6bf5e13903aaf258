"""Thin torch-facing layer over the native safetensors reader / writer (``csrc/host/safetensors_io.cpp``).

Reads go straight into caller-provided (pinned) host tensors with several concurrent ``pread`` streams, including row
ranges of dimension 0, which is what a rank needs to load only its shard of a parameter; writes lay the file out once
and fill tensors with parallel ``pwrite``.

Parity: csrc/src/utilities/safetensors.{h,cpp} (reader, writer, per-rank shard writes).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..ops import host

ST_TO_TORCH = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
               "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2}
TORCH_TO_ST = {v: k for k, v in ST_TO_TORCH.items()}


class NativeSafetensors:
    def __init__(self, path: str, threads: int = 8):
        self.path, self.threads = path, threads
        self._f = host().SafetensorsFile(path)
        self.entries: Dict[str, Tuple[str, list, int, int]] = dict(self._f.entries())

    def keys(self):
        return list(self.entries)

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def metadata(self) -> Dict[str, str]:
        return dict(self._f.metadata())

    def shape(self, name: str):
        return list(self.entries[name][1])

    def dtype(self, name: str) -> torch.dtype:
        return ST_TO_TORCH[self.entries[name][0]]

    def get_tensor(self, name: str, out: Optional[torch.Tensor] = None, pin: bool = False) -> torch.Tensor:
        st, shape, b, e = self.entries[name]
        if out is None:
            out = torch.empty(shape, dtype=ST_TO_TORCH[st], pin_memory=pin and torch.cuda.is_available())
        assert out.is_contiguous() and out.device.type == "cpu" and out.numel() * out.element_size() == e - b, "destination does not match the tensor"
        self._f.read_into(name, out.data_ptr(), e - b, 0, self.threads)
        return out

    def get_tensor_device(self, name: str, device, gds: Optional[bool] = None) -> torch.Tensor:
        """The tensor read straight into device memory: GPUDirect Storage (cuFile) when ``gds`` (default: the ``SUROGATE_GDS``
        variable) asks for it and it works on this machine, else pread into pinned double buffers overlapped with the
        host-to-device copies.  ``self.last_route`` says which route the last call took."""
        import os

        from ..ops import ext

        st, shape, b, e = self.entries[name]
        out = torch.empty(shape, dtype=ST_TO_TORCH[st], device=device)
        if e > b:
            want = os.environ.get("SUROGATE_GDS", "0") == "1" if gds is None else bool(gds)
            self.last_route = ext().read_file_to_device(self.path, self._f.data_start() + b, e - b, out, want)
        return out

    def get_rows(self, name: str, row_begin: int, row_end: int, out: Optional[torch.Tensor] = None, pin: bool = False) -> torch.Tensor:
        st, shape, _, _ = self.entries[name]
        if out is None:
            out = torch.empty([row_end - row_begin] + list(shape[1:]), dtype=ST_TO_TORCH[st], pin_memory=pin and torch.cuda.is_available())
        self._f.read_rows(name, out.data_ptr(), row_begin, row_end, self.threads)
        return out


def save_file_native(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None, threads: int = 8) -> int:
    items, keep = [], []
    for name in sorted(tensors):
        t = tensors[name].detach()
        if t.device.type != "cpu":
            t = t.cpu()
        t = t.contiguous()
        keep.append(t)
        items.append((name, TORCH_TO_ST[t.dtype], list(t.shape), t.data_ptr(), t.numel() * t.element_size()))
    return host().write_safetensors(path, items, dict(metadata or {}), threads)

"""Streaming data loader over token shard files.

Serves ``batch x seq_len`` int32 (inputs, targets, position_ids) per call.  Order is a two-level seeded
shuffle (files, then chunks inside a file) that depends only on (seed, epoch), so a run can be resumed
from ``state_dict()`` = (seed, epoch, file_index, chunk_index) and a rank can take every world-th chunk.
Targets are the inputs shifted by one; positions whose loss mask is 0 and the last position of a packed row
become -100.  The heavy lifting (mmap, shuffle, batch assembly on a prefetch thread) is done by the native
``TokenLoader`` (``csrc/host/token_loader.cpp``) when the host runtime is built; the numpy path below produces the
same batches in the same order and is what runs otherwise.

Parity: csrc/src/runtime/training/dataloader.{h,cpp} (DataLoader dataloader.h:39).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .tokfile import read_token_file

IGNORE = -100
_M64 = (1 << 64) - 1


def shuffled_order(n: int, seed: int, epoch: int, salt: int, shuffle: bool = True) -> np.ndarray:
    """Fisher-Yates driven by splitmix64: the same permutation as the native loader's ``shuffled_order``."""
    v = np.arange(n, dtype=np.int64)
    if not shuffle or n < 2:
        return v
    s = ((seed & _M64) * 0x9E3779B97F4A7C15 & _M64) ^ (((epoch + 0x1000) & _M64) * 0xC2B2AE3D27D4EB4F & _M64) ^ \
        (((salt + 0x2000) & _M64) * 0x165667B19E3779F9 & _M64)
    out = v.tolist()
    for i in range(n - 1, 0, -1):
        s = (s + 0x9E3779B97F4A7C15) & _M64
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
        z ^= z >> 31
        j = z % (i + 1)
        out[i], out[j] = out[j], out[i]
    return np.asarray(out, dtype=np.int64)


def _native():
    try:
        from ..ops import host

        return host()
    except Exception:  # noqa: BLE001
        return None


class DataLoader:
    def __init__(self, files: Sequence[str], batch: int, seq_len: int, seed: int = 0, rank: int = 0, world: int = 1, shuffle: bool = True,
                 native: Optional[bool] = None, prefetch: int = 2):
        if not files:
            raise ValueError("DataLoader needs at least one token file")
        self.files = list(files)
        self.batch, self.T, self.seed, self.rank, self.world, self.shuffle = batch, seq_len, seed, rank, world, shuffle
        mod = _native() if native in (None, True) else None
        if native is True and mod is None:
            raise RuntimeError("the native host runtime is not built")
        self._nat = mod.TokenLoader(self.files, batch, seq_len, seed, rank, world, shuffle, prefetch) if mod is not None else None
        self.epoch = 0
        self.file_index = 0
        self.chunk_index = 0
        self._cur = None
        self._file_order = self._order(len(self.files), salt=0)
        self.chunks_per_file = []
        for f in self.files:
            tok, _, _, h = read_token_file(f)
            self.chunks_per_file.append(self._chunks_in(h["n_tokens"], h["non_overlapping"]))
        self.total_chunks = sum(self.chunks_per_file)

    # a chunk = one row of T (+1 for the shifted target when rows overlap)
    def _chunks_in(self, n_tokens: int, non_overlapping: int) -> int:
        return n_tokens // self.T if non_overlapping else max(0, (n_tokens - 1) // self.T)

    def _order(self, n: int, salt: int) -> np.ndarray:
        return shuffled_order(n, self.seed, self.epoch, salt, self.shuffle)

    def _open(self, fi: int):
        path = self.files[self._file_order[fi]]
        tok, pos, mask, h = read_token_file(path)
        n = self._chunks_in(h["n_tokens"], h["non_overlapping"])
        order = self._order(n, salt=1 + int(self._file_order[fi]))
        order = order[self.rank::self.world]  # each rank walks its own residue class of the shuffled chunks
        self._cur = (tok, pos, mask, h, order)

    def steps_per_epoch(self) -> int:
        return sum(c // self.world for c in self.chunks_per_file) // self.batch

    def _advance_file(self):
        self.file_index += 1
        self.chunk_index = 0
        self._cur = None
        if self.file_index >= len(self.files):
            self.file_index = 0
            self.epoch += 1
            self._file_order = self._order(len(self.files), salt=0)

    def next_batch(self) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
        B, T = self.batch, self.T
        x = np.empty((B, T), np.int32)
        y = np.empty((B, T), np.int32)
        p = np.empty((B, T), np.int32)
        if self._nat is not None:
            self._nat.next_into(x.ctypes.data, y.ctypes.data, p.ctypes.data)
            st = self._nat.state()
            self.epoch, self.file_index, self.chunk_index = st["epoch"], st["file_index"], st["chunk_index"]
            return x, y, p
        row = 0
        guard = 0
        self.last_rows = []  # (file path, chunk index) of every row served: lets sidecar data (teacher log-probs) follow the batch
        while row < B:
            if self._cur is None:
                self._open(self.file_index)
            tok, pos, mask, h, order = self._cur
            if self.chunk_index >= len(order):
                self._advance_file()
                guard += 1
                if guard > 2 * len(self.files) + 2:
                    raise RuntimeError("token files hold fewer rows than one batch per rank")
                continue
            c = int(order[self.chunk_index])
            self.chunk_index += 1
            self.last_rows.append((self.files[self._file_order[self.file_index]], c))
            s = c * T
            x[row] = tok[s:s + T]
            p[row] = pos[s:s + T] if pos is not None else np.arange(T, dtype=np.int32)
            if h["non_overlapping"]:
                y[row, :-1] = tok[s + 1:s + T]
                y[row, -1] = IGNORE
                if pos is not None:  # a position reset marks the first token of the next packed document: not a target
                    y[row, :-1][p[row, 1:] == 0] = IGNORE
            else:
                y[row] = tok[s + 1:s + T + 1]
            if mask is not None:
                m = mask[s + 1:s + T + 1] if not h["non_overlapping"] else np.concatenate([mask[s + 1:s + T], [0]])
                y[row][m[:T] == 0] = IGNORE
            row += 1
        return x, y, p

    load_batch = next_batch

    def state_dict(self) -> Dict[str, int]:
        return {"seed": self.seed, "epoch": self.epoch, "file_index": self.file_index, "chunk_index": self.chunk_index}

    def load_state_dict(self, st: Dict[str, int]) -> None:
        self.seed, self.epoch = int(st["seed"]), int(st["epoch"])
        self.file_index, self.chunk_index = int(st["file_index"]), int(st["chunk_index"])
        self._file_order = self._order(len(self.files), salt=0)
        self._cur = None
        if self._nat is not None:
            self._nat.set_state(self.seed, self.epoch, self.file_index, self.chunk_index)

    def next_batch_pinned(self, x, y, p) -> None:
        """Native path: write the batch straight into caller-owned (pinned) int32 tensors of shape [batch, seq_len]."""
        if self._nat is None:
            a, b, c = self.next_batch()
            x.numpy()[...] = a
            y.numpy()[...] = b
            p.numpy()[...] = c
            return
        self._nat.next_into(x.data_ptr(), y.data_ptr(), p.data_ptr())
        st = self._nat.state()
        self.epoch, self.file_index, self.chunk_index = st["epoch"], st["file_index"], st["chunk_index"]


class DistillationFeed:
    """Teacher top-K log-probs (``.kd`` sidecars) for the rows a numpy-path ``DataLoader`` just served."""

    def __init__(self, loader: "DataLoader", sidecar_dir: Optional[str] = None):
        from ..distill.sidecar import SidecarReader, sidecar_path as _next_to_shard

        def sidecar_path(f):
            return os.path.join(sidecar_dir, os.path.basename(_next_to_shard(f))) if sidecar_dir else _next_to_shard(f)

        if loader._nat is not None:
            raise ValueError("distillation needs DataLoader(native=False): the sidecar rows follow the loader's row bookkeeping")
        self.loader = loader
        self.readers = {f: SidecarReader(sidecar_path(f)) for f in loader.files}
        self.K = next(iter(self.readers.values())).K

    def batch(self):
        T = self.loader.T
        idx = np.empty((len(self.loader.last_rows), T, self.K), np.int32)
        lp = np.empty((len(self.loader.last_rows), T, self.K), np.float32)
        for r, (f, c) in enumerate(self.loader.last_rows):
            idx[r], lp[r] = self.readers[f].rows(c * T, T)
        return idx, lp


def write_synthetic_tokens(path: str, n_rows: int, seq_len: int, vocab: int, seed: int = 0) -> str:
    """Uniform random token ids of the given shape, as a regular token shard (for benchmarks and tests)."""
    from .tokfile import TokenFileWriter

    rng = np.random.default_rng(seed)
    w = TokenFileWriter(path, vocab, has_masks=False, non_overlapping=True)
    for _ in range(n_rows):
        w.add(rng.integers(0, vocab, seq_len, dtype=np.int64).astype(np.int32))
    w.close()
    return path

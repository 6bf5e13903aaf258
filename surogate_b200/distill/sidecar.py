"""``.kd`` sidecar files: a teacher's top-K token log-probabilities, row-aligned with a token shard.

Layout: 1024-byte header of little-endian int32 — ``[0..1]`` magic ``"KD.LOGP\\n"``, ``[2]`` version (1), ``[3]`` K,
``[4]`` number of token positions N, ``[5]`` vocabulary size, ``[6]`` bytes per log-prob (2 = fp16, 4 = fp32),
``[7]`` temperature * 1000 — followed by int32 indices ``[N, K]`` and log-probs ``[N, K]``.  Position ``i`` describes the
teacher's distribution over the token *following* token ``i`` of the shard (i.e. it is aligned with the training target of
position ``i``), so a loader that serves rows ``[r*T, (r+1)*T)`` of the shard serves the same slice of the sidecar.

Parity: surogate/distill/sidecar.py (1024-byte header, "KD.LOGP\\n").
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import numpy as np

KD_MAGIC = b"KD.LOGP\n"
HEADER_BYTES = 1024


class SidecarWriter:
    def __init__(self, path: str, top_k: int, vocab_size: int, temperature: float = 1.0, fp16: bool = True):
        self.path, self.K, self.vocab, self.temp, self.fp16 = path, top_k, vocab_size, temperature, fp16
        self.idx, self.lp = [], []

    def add(self, indices: np.ndarray, logprobs: np.ndarray) -> None:
        assert indices.shape == logprobs.shape and indices.shape[-1] == self.K
        self.idx.append(np.asarray(indices, np.int32).reshape(-1, self.K))
        self.lp.append(np.asarray(logprobs, np.float32).reshape(-1, self.K))

    def close(self) -> int:
        idx = np.concatenate(self.idx) if self.idx else np.zeros((0, self.K), np.int32)
        lp = np.concatenate(self.lp) if self.lp else np.zeros((0, self.K), np.float32)
        h = np.zeros(HEADER_BYTES // 4, "<i4")
        h[0:2] = np.frombuffer(KD_MAGIC, "<i4")
        h[2], h[3], h[4], h[5], h[6], h[7] = 1, self.K, idx.shape[0], self.vocab, 2 if self.fp16 else 4, int(round(self.temp * 1000))
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        with open(self.path + ".tmp", "wb") as f:
            f.write(h.tobytes())
            f.write(idx.astype("<i4").tobytes())
            f.write(lp.astype("<f2" if self.fp16 else "<f4").tobytes())
        os.replace(self.path + ".tmp", self.path)
        return idx.shape[0]


class SidecarReader:
    def __init__(self, path: str):
        with open(path, "rb") as f:
            raw = f.read(HEADER_BYTES)
        if len(raw) < HEADER_BYTES or raw[:8] != KD_MAGIC:
            raise ValueError(f"{path}: not a KD sidecar (bad magic)")
        h = np.frombuffer(raw, "<i4")
        if h[2] != 1 or h[6] not in (2, 4):
            raise ValueError(f"{path}: unsupported sidecar version {h[2]} / width {h[6]}")
        self.path, self.K, self.N, self.vocab, self.temperature = path, int(h[3]), int(h[4]), int(h[5]), h[7] / 1000.0
        need = HEADER_BYTES + self.N * self.K * (4 + int(h[6]))
        if os.path.getsize(path) < need:
            raise ValueError(f"{path}: truncated sidecar")
        self.idx = np.memmap(path, "<i4", "r", HEADER_BYTES, (self.N, self.K))
        self.lp = np.memmap(path, "<f2" if h[6] == 2 else "<f4", "r", HEADER_BYTES + 4 * self.N * self.K, (self.N, self.K))

    def rows(self, start: int, count: int) -> Tuple[np.ndarray, np.ndarray]:
        return np.asarray(self.idx[start:start + count]), np.asarray(self.lp[start:start + count], np.float32)


def sidecar_path(shard_path: str) -> str:
    return os.path.splitext(shard_path)[0] + ".kd"

"""Token shard file format (``train-NNN.bin`` / ``eval.bin``), byte-compatible with the reference's files.

Layout: 1024-byte header of 256 little-endian int32 — ``[0..1]`` magic ``"BIN.TOK\\n"``, ``[2]`` version (3),
``[3]`` bytes per token (4), ``[4]`` number of tokens, ``[5]`` vocabulary size, ``[6]`` has_masks,
``[7]`` non_overlapping (rows are whole packed sequences) — followed by int32 token ids, (v3) int32
position ids and, when ``has_masks``, one loss-mask bit per token packed LSB-first.

Parity: surogate/train/tokenize.py:113-214 (writer), csrc/src/runtime/training/dataloader.cpp:183-217 (reader).
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import numpy as np

TOK_MAGIC = b"BIN.TOK\n"
HEADER_BYTES = 1024
VERSION = 3


class TokenFileWriter:
    def __init__(self, path: str, vocab_size: int, has_masks: bool = True, non_overlapping: bool = True):
        self.path, self.vocab, self.has_masks, self.non_overlapping = path, vocab_size, has_masks, non_overlapping
        self.tokens, self.positions, self.masks = [], [], []

    def add(self, tokens, position_ids=None, loss_mask=None) -> None:
        t = np.asarray(tokens, dtype=np.int32)
        self.tokens.append(t)
        self.positions.append(np.asarray(position_ids, dtype=np.int32) if position_ids is not None else np.arange(len(t), dtype=np.int32))
        self.masks.append(np.asarray(loss_mask, dtype=np.uint8) if loss_mask is not None else np.ones(len(t), dtype=np.uint8))

    def close(self) -> int:
        tok = np.concatenate(self.tokens) if self.tokens else np.zeros(0, np.int32)
        pos = np.concatenate(self.positions) if self.positions else np.zeros(0, np.int32)
        header = np.zeros(HEADER_BYTES // 4, dtype="<i4")
        header[0:2] = np.frombuffer(TOK_MAGIC, dtype="<i4")
        header[2], header[3], header[4], header[5] = VERSION, 4, len(tok), self.vocab
        header[6], header[7] = int(self.has_masks), int(self.non_overlapping)
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        with open(self.path, "wb") as f:
            f.write(header.tobytes())
            f.write(tok.astype("<i4").tobytes())
            f.write(pos.astype("<i4").tobytes())
            if self.has_masks:
                f.write(np.packbits(np.concatenate(self.masks) if self.masks else np.zeros(0, np.uint8), bitorder="little").tobytes())
        return len(tok)


def read_header(path: str) -> Dict[str, int]:
    with open(path, "rb") as f:
        raw = f.read(HEADER_BYTES)
    if len(raw) < HEADER_BYTES or raw[:8] != TOK_MAGIC:
        raise ValueError(f"{path}: not a token shard (bad magic)")
    h = np.frombuffer(raw, dtype="<i4")
    if h[2] < 1 or h[2] > VERSION or h[3] != 4:
        raise ValueError(f"{path}: unsupported version {h[2]} / bytes per token {h[3]}")
    return {"version": int(h[2]), "n_tokens": int(h[4]), "vocab": int(h[5]), "has_masks": int(h[6]), "non_overlapping": int(h[7])}


def read_token_file(path: str, mmap: bool = True):
    """Returns (tokens int32 [n], position_ids int32 [n] or None, mask uint8 [n] or None, header)."""
    h = read_header(path)
    n = h["n_tokens"]
    expected = HEADER_BYTES + 4 * n + (4 * n if h["version"] >= 3 else 0) + ((n + 7) // 8 if h["has_masks"] else 0)
    if os.path.getsize(path) < expected:
        raise ValueError(f"{path}: truncated ({os.path.getsize(path)} bytes, header implies {expected})")
    load = (lambda off, cnt, dt: np.memmap(path, dtype=dt, mode="r", offset=off, shape=(cnt,))) if mmap else \
        (lambda off, cnt, dt: np.fromfile(path, dtype=dt, count=cnt, offset=off))
    tok = load(HEADER_BYTES, n, "<i4")
    off = HEADER_BYTES + 4 * n
    pos = None
    if h["version"] >= 3:
        pos = load(off, n, "<i4")
        off += 4 * n
    mask = None
    if h["has_masks"]:
        bits = np.fromfile(path, dtype=np.uint8, count=(n + 7) // 8, offset=off)
        mask = np.unpackbits(bits, bitorder="little")[:n]
    return tok, pos, mask, h

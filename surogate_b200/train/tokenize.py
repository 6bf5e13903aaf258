"""Dataset -> token shards: tokenise, pack, write ``train-NNN.bin`` / ``eval.bin`` once and reuse them by content hash.

The hash covers everything that changes the bytes written (dataset configs, tokenizer files, sequence length, packing,
loss-scale mode, seeds, split ratio).  A ``manifest.json`` next to the shards records it; a later run with the same hash
skips tokenisation.  With ``sample_packing`` whole documents are placed first-fit-decreasing into rows of
``sequence_len`` tokens; position ids restart at 0 for every document (which is also what tells attention and the loss
where documents begin) and the remainder of a row is padding with the loss mask cleared.  Without packing every
document is truncated / padded to one row.

Parity: surogate/train/tokenize.py (TokenizedDataFileWriter :113-214, packing :242-290, TokenizeDatasets :537).
"""
from __future__ import annotations

import contextlib
import dataclasses
import glob
import hashlib
import json
import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..data.datasets import load_dataset_rows
from ..data.tokfile import TokenFileWriter

IGNORE = -100
LOSS_SCALE_MODES = {"default": "assistant", "all": "all", "last_round": "last"}


def loss_scale_mode(loss_scale: str) -> str:
    """``loss_scale`` -> the tokenizer's ``train_on``: ``default`` (assistant turns), ``last_round`` (the assistant turns after the last
    user message), ``all`` (every token); the ``<base>+<name>`` spelling is accepted with ``-`` / a base name as ``<name>``.  A message's
    own ``loss`` field (0 or 1) overrides the mode for that turn.  Parity: surogate/core/model/loss_scale/loss_scale.py."""
    base, _, name = (loss_scale or "default").partition("+")
    if base not in LOSS_SCALE_MODES:
        base, name = "default", base
    if name not in ("", "-", *LOSS_SCALE_MODES):
        raise ValueError(f"unknown loss_scale '{loss_scale}' (default | last_round | all)")
    return LOSS_SCALE_MODES[base]
ROWS_PER_SHARD = 1 << 14


def tokenizer_dir(cfg) -> Optional[str]:
    """Where the run's tokenizer lives: ``tokenizer_path`` when set, else the model directory, else the hub model's local copy."""
    explicit = getattr(cfg, "tokenizer_path", None)
    if explicit:
        return explicit
    m = cfg.model
    if not isinstance(m, str) or m.strip().startswith("{") or m.lower().startswith("preset:"):
        return None
    if os.path.isdir(m):
        return m
    try:
        from ..hub import download_model

        d = download_model(m)
        return d if os.path.isdir(d) else None
    except Exception:  # noqa: BLE001 - offline and not cached
        return None


@contextlib.contextmanager
def directory_lock(directory: str, name: str = ".tokenize.lock"):
    """Exclusive advisory lock on a file inside ``directory`` (held while shards are written, released on every way out)."""
    import fcntl

    path = os.path.join(directory, name)
    with open(path, "a+") as f:
        fcntl.flock(f, fcntl.LOCK_EX)
        try:
            yield path
        finally:
            fcntl.flock(f, fcntl.LOCK_UN)


def progress(rows, label: str):
    """The rows, with a progress bar on a terminal (tokenising a large dataset takes minutes); plain iteration elsewhere."""
    import sys

    if not sys.stderr.isatty() or os.environ.get("SUROGATE_NO_PROGRESS") == "1":
        return rows
    try:
        from tqdm import tqdm

        return tqdm(rows, desc=label, unit="row", leave=False)
    except ImportError:
        return rows


PARALLEL_MIN_ROWS = 8192   # below this a pool's start-up (each worker imports the package and loads the tokenizer) costs more than it saves
MAX_DATASET_PROCESSES = 8


def dataset_processes(cfg=None) -> int:
    """How many processes tokenise a dataset: ``dataloader_num_workers`` when set, else ``SUROGATE_DATASET_PROCESSES``, else
    ``RUNPOD_CPU_COUNT`` (containers whose ``os.cpu_count()`` shows the host's cores), else the core count; at most 8.

    Parity: surogate/core/config/train_dataset_config.py:9-15, :64."""
    n = int(getattr(cfg, "dataloader_num_workers", 0) or 0)
    if n <= 0:
        for var in ("SUROGATE_DATASET_PROCESSES", "RUNPOD_CPU_COUNT"):
            if os.environ.get(var):
                n = int(os.environ[var])
                break
        else:
            n = os.cpu_count() or 1
    return max(1, min(n, MAX_DATASET_PROCESSES))


_worker = None  # a pool worker's own TokenizeDatasets


def _worker_init(fields: Dict[str, Any], hf_config: Dict[str, Any], model_dir: str) -> None:
    import types

    from ..data.tokenizer import Tokenizer

    global _worker
    _worker = TokenizeDatasets(types.SimpleNamespace(**fields), hf_config, "", tokenizer=Tokenizer.from_pretrained(model_dir))


def _worker_encode(rows: List[Dict[str, Any]]) -> List[Optional[Tuple[np.ndarray, np.ndarray]]]:
    return [_worker.encode_kept(r) for r in rows]


def _file_digest(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()[:16]


def _dataset_fingerprint(ds) -> Dict[str, Any]:
    d = dataclasses.asdict(ds)
    p = ds.path
    if os.path.isfile(p):
        d["_content"] = _file_digest(p)
    elif os.path.isdir(p):
        d["_content"] = [(os.path.relpath(f, p), os.path.getsize(f), int(os.path.getmtime(f))) for f in sorted(glob.glob(os.path.join(p, "**", "*"), recursive=True))
                         if os.path.isfile(f)]
    return d


def pack_documents(docs: Sequence[Tuple[np.ndarray, np.ndarray]], seq_len: int, pad_id: int, packing: bool = True):
    """docs: (ids, loss_mask) per document -> rows of (ids, position_ids, mask), each exactly ``seq_len`` long."""
    rows: List[Tuple[np.ndarray, np.ndarray, np.ndarray]] = []
    if not packing:
        for ids, mask in docs:
            ids, mask = ids[:seq_len], mask[:seq_len]
            n = len(ids)
            row = np.full(seq_len, pad_id, np.int32)
            m = np.zeros(seq_len, np.uint8)
            row[:n], m[:n] = ids, mask
            pos = np.arange(seq_len, dtype=np.int32)
            rows.append((row, pos, m))
        return rows
    order = sorted(range(len(docs)), key=lambda i: -min(len(docs[i][0]), seq_len))
    bins: List[List[int]] = []
    space: List[int] = []
    for i in order:  # first-fit decreasing
        n = min(len(docs[i][0]), seq_len)
        if n == 0:
            continue
        for b, free in enumerate(space):
            if free >= n:
                bins[b].append(i)
                space[b] -= n
                break
        else:
            bins.append([i])
            space.append(seq_len - n)
    for members in bins:
        row = np.full(seq_len, pad_id, np.int32)
        pos = np.zeros(seq_len, np.int32)
        m = np.zeros(seq_len, np.uint8)
        at = 0
        for i in members:
            ids, mask = docs[i][0][:seq_len], docs[i][1][:seq_len]
            n = len(ids)
            row[at:at + n], m[at:at + n] = ids, mask
            pos[at:at + n] = np.arange(n)
            m[at] = 0  # the first token of a document is never a target (nothing precedes it)
            at += n
        pos[at:] = np.arange(seq_len - at)  # padding: its own "document" with the mask cleared
        rows.append((row, pos, m))
    return rows


class TokenizeDatasets:
    def __init__(self, cfg, hf_config: Dict[str, Any], out_dir: str, tokenizer=None):
        self.cfg, self.hf_config, self.out_dir = cfg, hf_config, out_dir
        self._tok = tokenizer
        self._tok_from_dir = tokenizer is None

    # ------------------------------------------------------------------ hashing / cache
    def tokenizer(self):
        if self._tok is None:
            from ..data.tokenizer import Tokenizer

            model_dir = tokenizer_dir(self.cfg)
            if model_dir is None:
                raise FileNotFoundError("tokenising datasets needs tokenizer.json: set `model:` to a model directory or a hub id, or `tokenizer_path:` "
                                        "next to an inline / preset model")
            self._tok = Tokenizer.from_pretrained(model_dir)
        return self._tok

    def content_hash(self) -> str:
        c = self.cfg
        tok_dir = tokenizer_dir(c)
        tok_files = {}
        if tok_dir:
            for name in ("tokenizer.json", "tokenizer_config.json", "chat_template.jinja"):
                p = os.path.join(tok_dir, name)
                if os.path.exists(p):
                    tok_files[name] = _file_digest(p)
        key = {"datasets": [_dataset_fingerprint(d) for d in c.datasets], "validation": [_dataset_fingerprint(d) for d in c.validation_datasets],
               "split": c.validation_split_ratio, "seq": c.sequence_len, "packing": c.sample_packing, "loss_scale": c.loss_scale,
               "chat": c.use_chat_template, "seeds": [c.train_seed, c.eval_seed], "tok": tok_files, "truncation": c.truncation_strategy, "format": 3}
        return hashlib.sha256(json.dumps(key, sort_keys=True, default=str).encode()).hexdigest()[:24]

    def _cached(self, h: str) -> Optional[Dict[str, List[str]]]:
        man = os.path.join(self.out_dir, "manifest.json")
        if not os.path.exists(man):
            return None
        with open(man) as f:
            m = json.load(f)
        files = {k: [os.path.join(self.out_dir, x) for x in v] for k, v in m.get("files", {}).items()}
        if m.get("hash") == h and all(os.path.exists(p) for v in files.values() for p in v):
            return files
        return None

    # ------------------------------------------------------------------ tokenisation
    def encode_row(self, row: Dict[str, Any]) -> Optional[Tuple[np.ndarray, np.ndarray]]:
        tok, c = self.tokenizer(), self.cfg
        if "text" in row:
            ids = tok.encode(row["text"])
            if tok.eos_token_id >= 0:
                ids = ids + [tok.eos_token_id]
            ids = np.asarray(ids, np.int32)
            return ids, np.ones(len(ids), np.uint8)
        if "messages" in row:
            if not c.use_chat_template:
                text = "\n".join(str(m["content"]) for m in row["messages"])
                ids = np.asarray(tok.encode(text) + ([tok.eos_token_id] if tok.eos_token_id >= 0 else []), np.int32)
                return ids, np.ones(len(ids), np.uint8)
            ids, labels = tok.encode_for_training(row["messages"], train_on=loss_scale_mode(c.loss_scale), tools=row.get("tools"))
            ids_a, lab = np.asarray(ids, np.int32), np.asarray(labels, np.int64)
            return ids_a, (lab != IGNORE).astype(np.uint8)
        return None

    def encode_kept(self, row: Dict[str, Any]) -> Optional[Tuple[np.ndarray, np.ndarray]]:
        """A row as (ids, mask) after truncation, or None when nothing of it trains (unknown shape, deleted, no trained token)."""
        enc = self.encode_row(row)
        if enc is None:
            return None
        enc = self._truncate(*enc)
        if enc is not None and len(enc[0]) > 1 and enc[1].any():
            return enc
        return None

    def encode_rows(self, rows: List[Dict[str, Any]], label: str = "tokenising") -> List[Tuple[np.ndarray, np.ndarray]]:
        """All rows, in order.  Large datasets go through a pool of processes (the chat template is rendered in Python, one core per
        process); each worker loads its own tokenizer from the model directory, so a tokenizer object handed in by the caller, or a
        small dataset, stays in this process."""
        n = dataset_processes(self.cfg)
        model_dir = tokenizer_dir(self.cfg) if self._tok_from_dir else None
        if n > 1 and model_dir and len(rows) >= PARALLEL_MIN_ROWS:
            import multiprocessing as mp

            c = self.cfg
            fields = {"use_chat_template": c.use_chat_template, "loss_scale": c.loss_scale, "sequence_len": c.sequence_len, "truncation_strategy": c.truncation_strategy}
            chunk = max(64, min(2048, len(rows) // (n * 8)))
            chunks = [rows[i:i + chunk] for i in range(0, len(rows), chunk)]
            out: List[Tuple[np.ndarray, np.ndarray]] = []
            # spawn, not fork: the parent may already hold CUDA and communicator state that a forked child must not touch
            with mp.get_context("spawn").Pool(n, initializer=_worker_init, initargs=(fields, self.hf_config, model_dir)) as pool:
                for part in progress(pool.imap(_worker_encode, chunks), f"{label} ({n} processes, chunks of {chunk})"):
                    out.extend(e for e in part if e is not None)
            return out
        return [e for e in (self.encode_kept(r) for r in progress(rows, label)) if e is not None]

    def _truncate(self, ids: np.ndarray, mask: np.ndarray):
        T = self.cfg.sequence_len
        if len(ids) <= T:
            return ids, mask
        if self.cfg.truncation_strategy == "left":
            return ids[-T:], mask[-T:]
        if self.cfg.truncation_strategy == "delete":
            return None
        return ids[:T], mask[:T]

    def _write(self, rows, prefix: str, vocab: int) -> List[str]:
        paths = []
        if prefix == "eval":
            chunks = [rows]
        else:
            chunks = [rows[i:i + ROWS_PER_SHARD] for i in range(0, len(rows), ROWS_PER_SHARD)] or [[]]
        for i, chunk in enumerate(chunks):
            name = "eval.bin" if prefix == "eval" else f"train-{i:03d}.bin"
            w = TokenFileWriter(os.path.join(self.out_dir, name), vocab, has_masks=True, non_overlapping=True)
            for ids, pos, m in chunk:
                w.add(ids, pos, m)
            w.close()
            paths.append(os.path.join(self.out_dir, name))
        return paths

    def run(self, write: bool = True) -> Dict[str, List[str]]:
        c = self.cfg
        h = self.content_hash()
        cached = self._cached(h)
        if cached is not None:
            return cached
        if not write:  # another rank writes; the caller synchronises and re-reads the manifest
            return {"train": [os.path.join(self.out_dir, "train-000.bin")], "eval": [os.path.join(self.out_dir, "eval.bin")]}
        os.makedirs(self.out_dir, exist_ok=True)
        with directory_lock(self.out_dir):   # two runs that share an output directory: the second waits, then finds the shards cached
            cached = self._cached(h)
            if cached is not None:
                return cached
            return self._tokenise(h)

    def _tokenise(self, h: str) -> Dict[str, List[str]]:
        c = self.cfg
        tok = self.tokenizer()
        pad = tok.pad_token_id if tok.pad_token_id >= 0 else 0

        def encode_all(datasets) -> List[Tuple[np.ndarray, np.ndarray]]:
            docs = []
            for ds in datasets:
                docs.extend(self.encode_rows(load_dataset_rows(ds), f"tokenising {os.path.basename(str(ds.path).rstrip('/')) or 'dataset'}"))
            return docs

        train_docs = encode_all(c.datasets)
        eval_docs = encode_all(c.validation_datasets)
        if not eval_docs and c.validation_split_ratio and len(train_docs) > 1:
            rng = np.random.default_rng(c.eval_seed)
            idx = rng.permutation(len(train_docs))
            n_eval = max(1, int(len(train_docs) * c.validation_split_ratio))
            eval_docs = [train_docs[i] for i in idx[:n_eval]]
            train_docs = [train_docs[i] for i in idx[n_eval:]]
        rng = np.random.default_rng(c.train_seed)
        train_docs = [train_docs[i] for i in rng.permutation(len(train_docs))]
        vocab = int(self.hf_config.get("vocab_size", tok.vocab_size))
        train_rows = pack_documents(train_docs, c.sequence_len, pad, c.sample_packing)
        eval_rows = pack_documents(eval_docs, c.sequence_len, pad, c.sample_packing)
        files = {"train": self._write(train_rows, "train", vocab), "eval": self._write(eval_rows, "eval", vocab) if eval_rows else []}
        stats = {"train_documents": len(train_docs), "eval_documents": len(eval_docs), "train_rows": len(train_rows), "eval_rows": len(eval_rows),
                 "train_tokens": int(sum(len(d[0]) for d in train_docs)), "trained_tokens": int(sum(int(d[1].sum()) for d in train_docs)),
                 "packing_efficiency": float(sum(min(len(d[0]), c.sequence_len) for d in train_docs) / max(1, len(train_rows) * c.sequence_len))}
        with open(os.path.join(self.out_dir, "manifest.json"), "w") as f:
            json.dump({"hash": h, "files": {k: [os.path.basename(p) for p in v] for k, v in files.items()}, "stats": stats}, f, indent=1)
        self.stats = stats
        return files

"""``surogate tokenize config.yaml``: run only the dataset -> token shard stage of a training config.

Parity: surogate/cli (tokenize command), surogate/train/tokenize.py:537.
"""
from __future__ import annotations

import argparse
import json
import os


def main(argv, command: str = "tokenize") -> int:
    p = argparse.ArgumentParser(prog="surogate tokenize")
    p.add_argument("config")
    p.add_argument("--output-dir", default=None, dest="output_dir")
    p.add_argument("--debug", action="store_true", help="print the tokens of the first rows with their labels, to check what the loss ignores")
    p.add_argument("--hub_token", "--hub-token", dest="hub_token", default=None)
    a = p.parse_args(argv)
    if a.hub_token:
        os.environ["HF_TOKEN"] = a.hub_token
    from ..config.loader import load_config
    from ..config.sft_config import SFTConfig
    from ..train.sft import resolve_model_config
    from ..train.tokenize import TokenizeDatasets

    cfg = load_config(SFTConfig, a.config, output_dir=a.output_dir)
    job = TokenizeDatasets(cfg, resolve_model_config(cfg), os.path.join(cfg.output_dir, "tokens"))
    files = job.run(write=True)
    print(json.dumps({"files": files, "stats": getattr(job, "stats", "cached")}))
    if a.debug and files.get("train"):
        print(debug_rows(files["train"][0], cfg.model if isinstance(cfg.model, str) else None, cfg.sequence_len))
    return 0


def debug_rows(shard: str, model_dir, seq_len: int, rows: int = 2) -> str:
    """The first rows of a shard, token by token: ``id 'text' label``; tokens the loss ignores are marked ``-``."""
    import numpy as np

    from ..data.tokfile import read_token_file

    tok, _pos, mask, h = read_token_file(shard)
    decode = None
    if model_dir and os.path.isdir(model_dir) and os.path.exists(os.path.join(model_dir, "tokenizer.json")):
        from ..data.tokenizer import Tokenizer

        decode = Tokenizer.from_pretrained(model_dir).decode
    lines = []
    for r in range(min(rows, h["n_tokens"] // seq_len)):
        ids = np.asarray(tok[r * seq_len:(r + 1) * seq_len])
        m = np.asarray(mask[r * seq_len:(r + 1) * seq_len]) if mask is not None else np.ones(seq_len, np.uint8)
        lines.append(f"--- row {r}: {int(m.sum())} of {seq_len} tokens trained")
        for i, t in enumerate(ids):
            text = repr(decode([int(t)])) if decode else ""
            lines.append(f"{i:6d} {int(t):8d} {text:24s} {'train' if m[i] else '-'}")
    return "\n".join(lines)

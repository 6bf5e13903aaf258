"""``surogate debug {weights,registry,activations,gradients,diff,determinism,sanitize,tensor-arena,tensor-layout,tensor-aliasing,tensor-resolve}``.

Parity: surogate/cli/debug.py."""
from __future__ import annotations

import argparse
import json

import numpy as np


def main(argv, command: str = "debug") -> int:
    p = argparse.ArgumentParser(prog="surogate debug")
    sub = p.add_subparsers(dest="what", required=True)
    sub.add_parser("sanitize", help="run the C++ host runtime under AddressSanitizer + UBSan")
    for name in ("weights", "registry", "activations", "gradients", "diff", "determinism"):
        s = sub.add_parser(name)
        s.add_argument("model", nargs="?" if name == "registry" else None, help="model directory (or architecture name for `registry`)")
        s.add_argument("--out", default=None, help="JSONL report path")
        s.add_argument("--seq-len", type=int, default=128)
        s.add_argument("--batch", type=int, default=1)
        s.add_argument("--seed", type=int, default=0)
    for name in ("tensor-arena", "tensor-layout", "tensor-aliasing", "tensor-resolve"):
        s = sub.add_parser(name, help="compile-only introspection of the buffer plan (no weights, no GPU)")
        s.add_argument("model", help="model directory or config.json")
        s.add_argument("--out", default=None)
        s.add_argument("--seq-len", type=int, default=2048)
        s.add_argument("--batch", type=int, default=1)
        if name == "tensor-arena":
            s.add_argument("--recompute", action="store_true")
        if name == "tensor-aliasing":
            s.add_argument("--mode", choices=["static", "runtime"], default="static")
        if name == "tensor-resolve":
            s.add_argument("--name", required=True)
    a = p.parse_args(argv)
    if a.what.startswith("tensor-"):
        from ..debug import tensor_tools as tt

        if a.what == "tensor-arena":
            rows = tt.tensor_arena(a.model, a.batch, a.seq_len, a.recompute, a.out)
        elif a.what == "tensor-layout":
            rows = tt.tensor_layout(a.model, a.batch, a.seq_len, a.out)
        elif a.what == "tensor-aliasing":
            rows = tt.tensor_aliasing(a.model, a.batch, min(a.seq_len, 256) if a.mode == "runtime" else a.seq_len, a.mode, a.out)
        else:
            rows = tt.tensor_resolve(a.model, a.name, a.batch, a.seq_len, a.out)
        tt.main_json(rows)
        return 0
    if a.what == "sanitize":
        from ..debug.sanitize import run

        return run([])
    from ..debug import tools

    if a.what == "weights":
        print(json.dumps(tools.audit_weights(a.model, a.out), indent=1))
        return 0
    if a.what == "registry":
        for r in tools.registry_report(a.model, a.out)[:4]:
            print(json.dumps(r)[:2000])
        return 0
    import torch

    from ..dsl.compiler import load_hf_config
    from ..runtime.trainer import Trainer, TrainerConfig

    cfg = load_hf_config(a.model)
    rng = np.random.default_rng(a.seed)
    tok = rng.integers(0, cfg.get("vocab_size", 1000), (a.batch, a.seq_len + 1)).astype(np.int32)
    if a.what == "determinism":
        dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")

        def make():
            tr = Trainer(TrainerConfig(model=cfg, batch_size=a.batch, seq_len=a.seq_len, zero_level=0), device=dev)
            tr.import_weights(a.model)
            return tr

        print(json.dumps(tools.determinism_report(make, tok[:, :-1], tok[:, 1:], out=a.out), indent=1))
        return 0
    if a.what == "diff":
        rows = tools.diff_against_transformers(a.model, tok[:, :-1], "cuda" if torch.cuda.is_available() else "cpu", a.out)
    else:
        dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
        tr = Trainer(TrainerConfig(model=cfg, batch_size=a.batch, seq_len=a.seq_len, zero_level=0), device=dev)
        tr.import_weights(a.model)
        fn = tools.activation_stats if a.what == "activations" else tools.gradient_stats
        rows = fn(tr, tok[:, :-1], tok[:, 1:], a.out)
    for r in rows[:20]:
        print(json.dumps(r))
    return 0

"""``surogate debug {weights,registry,activations,gradients,diff,determinism,sanitize,tensor-arena,tensor-layout,tensor-aliasing,tensor-resolve}``.

The positional argument is a model directory (or ``config.json``), or a training config in the format of ``surogate sft``: then the
model, sequence length and micro-batch come from the config (``--seq-len`` / ``--batch`` override), as do LoRA and recipe for the
tracing commands.

Parity: surogate/cli/debug.py."""
from __future__ import annotations

import argparse
import json

import numpy as np


def resolve_target(arg, seq_len=None, batch=None, default_seq: int = 128):
    """(model directory, seq_len, batch, training config or None) from a model path or a training config file."""
    import os

    cfg = None
    if arg and os.path.isfile(arg) and arg.lower().endswith((".yaml", ".yml")):
        from ..config.loader import load_config
        from ..config.sft_config import SFTConfig

        cfg = load_config(SFTConfig, arg)
        model = cfg.model
        if isinstance(model, str) and not os.path.exists(model) and not model.strip().startswith("{"):
            from ..hub import download_model

            model = download_model(model)
        return model, seq_len or min(cfg.sequence_len, 2048), batch or cfg.per_device_train_batch_size, cfg
    return arg, seq_len or default_seq, batch or 1, None


def main(argv, command: str = "debug") -> int:
    p = argparse.ArgumentParser(prog="surogate debug")
    sub = p.add_subparsers(dest="what", required=True)
    sub.add_parser("sanitize", help="run the C++ host runtime under AddressSanitizer + UBSan")
    for name in ("weights", "registry", "activations", "gradients", "diff", "determinism"):
        s = sub.add_parser(name)
        s.add_argument("model", nargs="?" if name == "registry" else None, help="model directory, or a training config (architecture name for `registry`)")
        s.add_argument("--out", "--output", dest="out", default=None, help="JSONL report path")
        s.add_argument("--seq-len", "--max-tokens", dest="seq_len", type=int, default=None)
        s.add_argument("--batch", type=int, default=None)
        s.add_argument("--seed", type=int, default=0)
        s.add_argument("--hub_token", "--hub-token", dest="hub_token", default=None)
        if name == "gradients":
            s.add_argument("--steps", type=int, default=1, help="forward + backward + optimizer cycles to run, gradients captured at each")
        if name == "diff":
            s.add_argument("--reference", default=None, help="the transformers model to compare with (default: the model itself)")
            s.add_argument("--rtol", type=float, default=1e-2)
            s.add_argument("--atol", type=float, default=1e-3)
    for name in ("tensor-arena", "tensor-layout", "tensor-aliasing", "tensor-resolve"):
        s = sub.add_parser(name, help="compile-only introspection of the buffer plan (no weights, no GPU)")
        s.add_argument("model", help="model directory, config.json, or a training config")
        s.add_argument("--out", "--output", dest="out", default=None)
        s.add_argument("--seq-len", type=int, default=None)
        s.add_argument("--batch", type=int, default=None)
        s.add_argument("--hub_token", "--hub-token", dest="hub_token", default=None)
        if name == "tensor-arena":
            s.add_argument("--recompute", action="store_true")
        if name == "tensor-aliasing":
            s.add_argument("--mode", choices=["static", "runtime"], default="static")
        if name == "tensor-resolve":
            s.add_argument("--name", required=True)
    a = p.parse_args(argv)
    if getattr(a, "hub_token", None):
        import os

        os.environ["HF_TOKEN"] = a.hub_token
    train_cfg = None
    if a.what != "sanitize" and getattr(a, "model", None):
        a.model, a.seq_len, a.batch, train_cfg = resolve_target(a.model, a.seq_len, a.batch, 2048 if a.what.startswith("tensor-") else 128)
    elif a.what != "sanitize":
        a.seq_len, a.batch = a.seq_len or 128, a.batch or 1
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
        rows = tools.diff_against_transformers(a.model, tok[:, :-1], "cuda" if torch.cuda.is_available() else "cpu", a.out, reference=a.reference, rtol=a.rtol, atol=a.atol)
    else:
        dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
        if train_cfg is not None:  # trace the model as the run would build it (LoRA, recipe, QLoRA)
            tc = train_cfg.to_trainer_config(cfg)
            tc.batch_size, tc.seq_len, tc.grad_accum, tc.zero_level = a.batch, a.seq_len, 1, 0
        else:
            tc = TrainerConfig(model=cfg, batch_size=a.batch, seq_len=a.seq_len, zero_level=0)
        tr = Trainer(tc, device=dev)
        tr.import_weights(a.model)
        if tr.lora is not None:
            tr.lora.init_weights(a.seed)
        if a.what == "activations":
            rows = tools.activation_stats(tr, tok[:, :-1], tok[:, 1:], a.out)
        else:
            rows = tools.gradient_stats(tr, tok[:, :-1], tok[:, 1:], a.out, steps=a.steps)
    for r in rows[:20]:
        print(json.dumps(r))
    return 0

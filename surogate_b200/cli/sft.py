"""``surogate sft config.yaml``.  Parity: surogate/cli/sft.py:13-25."""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys


def build_parser(prog: str) -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog=f"surogate {prog}")
    p.add_argument("config", help="YAML config (path or http(s) URL)")
    p.add_argument("--gpus", type=int, default=None, help="override `gpus`; > 1 re-launches under torch.distributed.run")
    p.add_argument("--max-steps", type=int, default=None, dest="max_steps")
    p.add_argument("--output-dir", default=None, dest="output_dir")
    p.add_argument("--model", default=None)
    p.add_argument("--recipe", default=None, help="override `recipe` (bf16 | fp8-hybrid | nvfp4)")
    p.add_argument("--synthetic-data", action="store_true", default=None, dest="synthetic_data")
    p.add_argument("--hub_token", "--hub-token", dest="hub_token", default=None, help="HuggingFace token for private models and datasets")
    return p


def take_hub_token(args) -> None:
    """``--hub_token`` reaches the hub helpers through ``HF_TOKEN``; it is not a config key."""
    token = getattr(args, "hub_token", None)
    if token:
        os.environ["HF_TOKEN"] = token
    if hasattr(args, "hub_token"):
        del args.hub_token


def launch(args, command: str, entry) -> int:
    from ..config.loader import read_yaml

    take_hub_token(args)
    overrides = {k: v for k, v in vars(args).items() if k != "config" and v is not None}
    gpus = overrides.get("gpus") or read_yaml(args.config).get("gpus", 1)
    if gpus > 1 and "RANK" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
               "--master-port", os.environ.get("MASTER_PORT", "29500"), "-m", "surogate_b200.cli.main", command] + sys.argv[2:]
        return subprocess.call(cmd)
    result = entry(args.config, **overrides)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"steps": result["steps"], "final": result["final"]}))
    return 0


def main(argv, command: str = "sft") -> int:
    from ..train.sft import sft_main

    return launch(build_parser(command).parse_args(argv), command, sft_main)

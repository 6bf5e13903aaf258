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
    a = p.parse_args(argv)
    from ..config.loader import load_config
    from ..config.sft_config import SFTConfig
    from ..train.sft import resolve_model_config
    from ..train.tokenize import TokenizeDatasets

    cfg = load_config(SFTConfig, a.config, output_dir=a.output_dir)
    job = TokenizeDatasets(cfg, resolve_model_config(cfg), os.path.join(cfg.output_dir, "tokens"))
    files = job.run(write=True)
    print(json.dumps({"files": files, "stats": getattr(job, "stats", "cached")}))
    return 0

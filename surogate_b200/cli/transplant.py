"""``surogate transplant-tokenizer``: give a model another model's tokenizer (wraps ``mergekit-tokensurgeon``).

Parity: surogate/transplant/transplant.py.
"""
from __future__ import annotations

import argparse
import shutil
import subprocess
import sys


def build_command(model: str, donor: str, output: str, approximation: str = "omp", k: int = 64, extra=None):
    return ["mergekit-tokensurgeon", model, donor, output, "--approximation-method", approximation, "-k", str(k)] + list(extra or [])


def main(argv, command: str = "transplant-tokenizer") -> int:
    p = argparse.ArgumentParser(prog="surogate transplant-tokenizer")
    p.add_argument("--model", required=True)
    p.add_argument("--donor", required=True, help="model whose tokenizer is transplanted")
    p.add_argument("--output", required=True)
    p.add_argument("--approximation", default="omp")
    p.add_argument("-k", type=int, default=64)
    a, extra = p.parse_known_args(argv)
    cmd = build_command(a.model, a.donor, a.output, a.approximation, a.k, extra)
    if shutil.which(cmd[0]) is None:
        print(f"`{cmd[0]}` is not installed (pip install mergekit); the command would be:\n  " + " ".join(cmd), file=sys.stderr)
        return 3
    return subprocess.call(cmd)

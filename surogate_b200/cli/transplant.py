"""``surogate transplant-tokenizer``: give a student model the teacher's tokenizer (cross-tokenizer distillation), and back.

    surogate transplant-tokenizer --student S --teacher T --output OUT [--method omp] [--k 64] [--device cuda] [--engine auto|builtin|mergekit]
    surogate transplant-tokenizer --restore OUT/transplant_manifest.json --student DISTILLED --output BACK

Parity: surogate/cli/transplant.py, surogate/transplant/transplant.py.
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv, command: str = "transplant-tokenizer") -> int:
    p = argparse.ArgumentParser(prog="surogate transplant-tokenizer")
    p.add_argument("--student", "--model", dest="student", help="student model directory or hub id (the model to be trained); with --restore: the distilled model")
    p.add_argument("--teacher", "--donor", dest="teacher", help="teacher model directory or hub id (the tokenizer donor)")
    p.add_argument("--output", required=True, help="output directory of the transplanted model")
    p.add_argument("--method", "--approximation", dest="method", default="omp", help="approximation of rows for new tokens (default omp)")
    p.add_argument("--k", "-k", dest="k", type=int, default=64, help="sparsity / neighbour count of the approximation")
    p.add_argument("--device", default=None, help="device of the approximation solve (e.g. cuda)")
    p.add_argument("--trust-remote-code", action="store_true", help="passed on to mergekit-tokensurgeon")
    p.add_argument("--engine", default="auto", choices=["auto", "builtin", "mergekit"], help="built-in PyTorch implementation or the external mergekit tool")
    p.add_argument("--restore", metavar="MANIFEST", default=None, help="reverse mode: a transplant_manifest.json; moves --student back to the original tokenizer")
    a, extra = p.parse_known_args(argv)
    from ..utils.tokenizer_transplant import run_transplant, run_transplant_back

    try:
        if a.restore:
            if not a.student:
                p.error("--restore needs --student (the distilled model to convert back)")
            res = run_transplant_back(a.student, a.restore, a.output, a.device, a.trust_remote_code, extra, a.engine)
        else:
            if not a.student or not a.teacher:
                p.error("give --student and --teacher (or --restore MANIFEST)")
            res = run_transplant(a.student, a.teacher, a.output, a.method, a.k, a.device, a.trust_remote_code, extra, a.engine)
    except (RuntimeError, ValueError) as e:
        print(f"transplant failed: {e}", file=sys.stderr)
        return 3
    print(json.dumps(res))
    return 0

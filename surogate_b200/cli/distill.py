"""``surogate distill-capture``: write teacher top-K log-prob sidecars next to token shards.

Parity: surogate/cli (distill-capture), surogate/distill/capture.py.
"""
from __future__ import annotations

import argparse
import glob
import json
import os


def main(argv, command: str = "distill-capture") -> int:
    p = argparse.ArgumentParser(prog="surogate distill-capture")
    p.add_argument("--tokens", required=True, help="directory with train-NNN.bin shards")
    p.add_argument("--teacher", required=True, help="HF model directory, or http(s)://host/v1 of an OpenAI-compatible server")
    p.add_argument("--teacher-model", default=None, help="model name for an API teacher")
    p.add_argument("--sequence-len", type=int, required=True)
    p.add_argument("--top-k", type=int, default=64)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--rows-per-call", type=int, default=4)
    p.add_argument("--workers", type=int, default=8, help="concurrent requests to an API teacher")
    p.add_argument("--no-resume", action="store_true", help="capture again even where a complete sidecar exists")
    a = p.parse_args(argv)
    from ..data.tokfile import read_header
    from ..distill.capture import api_teacher_rows, capture, hf_teacher

    shards = sorted(glob.glob(os.path.join(a.tokens, "train-*.bin")))
    if not shards:
        raise SystemExit(f"no train-*.bin under {a.tokens}")
    vocab = read_header(shards[0])["vocab"]
    teacher = direct = None
    if a.teacher.startswith(("http://", "https://")):
        direct = api_teacher_rows(a.teacher, a.teacher_model or "teacher", a.top_k, workers=a.workers)
    else:
        import torch

        teacher = hf_teacher(a.teacher, "cuda" if torch.cuda.is_available() else "cpu")
    out = capture(shards, teacher, a.sequence_len, a.top_k, vocab, resume=not a.no_resume, temperature=a.temperature, rows_per_call=a.rows_per_call, direct=direct)
    print(json.dumps({"sidecars": out}))
    return 0

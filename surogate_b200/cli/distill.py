"""``surogate distill-capture``: write teacher top-K log-prob sidecars (``train-NNN.kd``) for the token shards of a run.

    surogate distill-capture config.yaml [--api-base http://host:8000/v1] [--device cuda:0]
    surogate distill-capture --tokens DIR --teacher MODEL_OR_URL --sequence-len T [--top-k K] ...

With a config the command tokenises the datasets exactly as the training run will (same shard directory, same content hash), takes
teacher, K, temperature and the API settings from the ``distillation`` section, and writes each sidecar next to its shard (or
into ``distillation.kd_dir``).  Complete sidecars are kept, so an interrupted capture resumes.

Parity: surogate/cli/distill_capture.py, surogate/distill/capture.py.
"""
from __future__ import annotations

import argparse
import glob
import json
import os


def main(argv, command: str = "distill-capture") -> int:
    p = argparse.ArgumentParser(prog="surogate distill-capture")
    p.add_argument("config", nargs="?", help="training config with a `distillation` section (path or URL)")
    p.add_argument("--api-base", default=None, help="OpenAI-compatible base URL of a served teacher (overrides distillation.teacher_api_base)")
    p.add_argument("--device", default=None, help="device of a local teacher (default cuda:0, cpu without a GPU)")
    p.add_argument("--tokens", default=None, help="without a config: directory with train-NNN.bin shards")
    p.add_argument("--teacher", default=None, help="without a config: HF model directory, or http(s)://host/v1 of an OpenAI-compatible server")
    p.add_argument("--teacher-model", default=None, help="model name for an API teacher")
    p.add_argument("--sequence-len", type=int, default=None)
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--temperature", type=float, default=None)
    p.add_argument("--rows-per-call", type=int, default=None)
    p.add_argument("--workers", type=int, default=None, help="concurrent requests to an API teacher")
    p.add_argument("--no-resume", action="store_true", help="capture again even where a complete sidecar exists")
    a = p.parse_args(argv)
    from ..data.tokfile import read_header
    from ..distill.capture import api_teacher_rows, capture, hf_teacher

    out_dir, api_key, timeout = None, "EMPTY", 600.0
    if a.config:
        from ..config.loader import load_config
        from ..config.sft_config import SFTConfig
        from ..train.sft import prepare_data, resolve_model_config

        cfg = load_config(SFTConfig, a.config)
        d = cfg.distillation
        if d is None:
            raise SystemExit("the config has no `distillation` section")
        shards = prepare_data(cfg, resolve_model_config(cfg), rank=0)["train"]
        api_base = a.api_base or d.teacher_api_base
        teacher_name = a.teacher_model or a.teacher or d.teacher
        seq_len, top_k, temperature = a.sequence_len or cfg.sequence_len, a.top_k or d.top_k, a.temperature or d.temperature
        rows, workers, out_dir, api_key, timeout = a.rows_per_call or d.teacher_batch_size, a.workers or d.teacher_api_concurrency, d.sidecar_dir, d.api_key(), float(d.teacher_api_timeout)
    else:
        if not (a.tokens and a.teacher and a.sequence_len):
            p.error("give a config, or --tokens, --teacher and --sequence-len")
        shards = sorted(glob.glob(os.path.join(a.tokens, "train-*.bin")))
        is_url = a.teacher.startswith(("http://", "https://"))
        api_base = a.api_base or (a.teacher if is_url else None)
        teacher_name = a.teacher_model or (None if is_url else a.teacher)
        seq_len, top_k, temperature, rows, workers = a.sequence_len, a.top_k or 64, a.temperature or 1.0, a.rows_per_call or 4, a.workers or 8
    if not shards:
        raise SystemExit("no train-*.bin token shards to capture")
    if not api_base and not teacher_name:
        raise SystemExit("no teacher: set distillation.teacher (or teacher_model), or --api-base")
    vocab = read_header(shards[0])["vocab"]
    teacher = direct = None
    if api_base:
        if a.device:
            print("--device is ignored with an API teacher")
        direct = api_teacher_rows(api_base, teacher_name or "teacher", top_k, timeout_s=timeout, workers=workers, api_key=api_key)
    else:
        import torch

        teacher = hf_teacher(teacher_name, a.device or ("cuda:0" if torch.cuda.is_available() else "cpu"))
    out = capture(shards, teacher, seq_len, top_k, vocab, resume=not a.no_resume, temperature=temperature, rows_per_call=rows, direct=direct, out_dir=out_dir)
    print(json.dumps({"sidecars": out}))
    return 0

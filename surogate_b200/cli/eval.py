"""``surogate eval config.yaml [--checkpoint dir] [--adapter dir] [--batches N]``: validation loss and perplexity.

Loads the model of the config (HF directory, optionally the latest or a given training checkpoint, optionally a LoRA adapter),
tokenises the config's validation data the same way training does (cached) and averages the next-token loss over ``--batches``
batches of the evaluation shard.

Parity: the evaluation pass of surogate/train/trainer.py (eval_steps) as a stand-alone command.
"""
from __future__ import annotations

import argparse
import glob
import json
import math
import os


def main(argv, command: str = "eval") -> int:
    p = argparse.ArgumentParser(prog="surogate eval")
    p.add_argument("config")
    p.add_argument("--checkpoint", default=None, help="training checkpoint directory (latest step); default: the model's own weights")
    p.add_argument("--adapter", default=None, help="PEFT adapter directory to load on top")
    p.add_argument("--batches", type=int, default=16)
    p.add_argument("--synthetic-data", action="store_true")
    a = p.parse_args(argv)
    import torch

    from ..config.loader import load_config
    from ..config.sft_config import SFTConfig
    from ..data.loader import DataLoader
    from ..runtime.trainer import Trainer
    from ..train.sft import prepare_data, resolve_model_config

    cfg = load_config(SFTConfig, a.config, **({"synthetic_data": True} if a.synthetic_data else {}))
    hf = resolve_model_config(cfg)
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    tr = Trainer(cfg.to_trainer_config(hf), device=dev)
    model_dir = cfg.model if isinstance(cfg.model, str) and os.path.isdir(cfg.model) else None
    if a.checkpoint:
        tr.load_checkpoint(a.checkpoint)
    elif model_dir and glob.glob(os.path.join(model_dir, "*.safetensors")):
        tr.import_weights(model_dir)
    else:
        tr.init_weights(cfg.train_seed)
    if a.adapter and tr.lora is not None:
        tr.lora.load_peft(a.adapter)
    files = prepare_data(cfg, hf, 0)
    if not files.get("eval"):
        raise SystemExit("the config defines no validation data (validation_datasets or validation_split_ratio)")
    loader = DataLoader(files["eval"], cfg.per_device_train_batch_size, cfg.sequence_len, seed=cfg.eval_seed, shuffle=False)
    n = max(1, min(a.batches, loader.steps_per_epoch()))
    total = 0.0
    for _ in range(n):
        x, y, _pos = loader.next_batch()
        total += tr.validate(x, y)["loss"]
    loss = total / n
    print(json.dumps({"eval_loss": loss, "perplexity": math.exp(min(loss, 50.0)), "batches": n, "tokens_per_batch": cfg.per_device_train_batch_size * cfg.sequence_len}))
    return 0

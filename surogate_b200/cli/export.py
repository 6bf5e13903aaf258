"""``surogate export --checkpoint <dir> --output <dir>``: turn a training checkpoint into an HF model directory.

Parity: MultiGPUPyTrainer.export_model (csrc/src/binding/py_train.h).
"""
from __future__ import annotations

import argparse
import json
import os


def main(argv, command: str = "export") -> int:
    p = argparse.ArgumentParser(prog="surogate export")
    p.add_argument("config", help="the training config the checkpoint was written with")
    p.add_argument("--checkpoint", default=None, help="checkpoint directory (default: the config's checkpoint_dir, latest step)")
    p.add_argument("--output", required=True)
    p.add_argument("--push-to-hub", default=None, metavar="REPO_ID", help="upload the exported directory to this model repository afterwards")
    p.add_argument("--private", action="store_true")
    p.add_argument("--hub_token", "--hub-token", dest="hub_token", default=None)
    a = p.parse_args(argv)
    import torch

    from ..config.loader import load_config
    from ..config.sft_config import SFTConfig
    from ..runtime.trainer import Trainer
    from ..train.sft import resolve_model_config

    cfg = load_config(SFTConfig, a.config)
    hf = resolve_model_config(cfg)
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    tr = Trainer(cfg.to_trainer_config(hf), device=dev)
    meta = tr.load_checkpoint(a.checkpoint or cfg.checkpoint_dir)
    if tr.lora is not None:
        tr.export_adapter(os.path.join(a.output, "adapter"), base_model=cfg.model if isinstance(cfg.model, str) else "")
        tr.lora.merge_into(tr.store)
    tr.export_model(a.output, hf)
    out = {"step": meta["run"]["step"], "output": a.output}
    if a.push_to_hub:
        from ..hub import push_to_hub

        push_to_hub(a.push_to_hub, a.output, private=a.private, token=a.hub_token, commit_message=f"step {meta['run']['step']}")
        out["pushed_to"] = a.push_to_hub
    print(json.dumps(out))
    return 0

"""Starting a run from an existing adapter (``adapter_path`` + ``adapter_init_mode``).

* ``merge``  — fold the adapter into the base weights, then train fresh adapters on top (continual fine-tuning);
* ``resume`` / ``trainable`` — load the adapter into the trainable LoRA weights and keep training it; ``trainable`` also checks that
  the adapter's rank, alpha and target modules are those of this run, and that its two files are complete;
* ``stack``  — like merge, but the old adapter is also kept in the output for reference.

Parity: surogate/train/adapter_init.py.
"""
from __future__ import annotations

import os
import shutil


def apply_adapter_init(trainer, adapter_path: str, mode: str = "merge", output_dir: str = "") -> str:
    if trainer.lora is None:
        raise ValueError("adapter_path needs lora: true")
    if mode not in ("merge", "resume", "trainable", "stack"):
        raise ValueError(f"[E140] adapter_init_mode must be merge | trainable | resume | stack, got '{mode}'")
    missing = [n for n in ("adapter_config.json", "adapter_model.safetensors") if not os.path.isfile(os.path.join(adapter_path, n))]
    if missing:
        raise FileNotFoundError(f"initial adapter is incomplete at {adapter_path}: missing {', '.join(missing)}")
    if mode == "trainable":
        import json

        with open(os.path.join(adapter_path, "adapter_config.json")) as f:
            ac = json.load(f)
        lc = trainer.cfg.lora or {}
        if int(ac.get("r", -1)) != int(lc.get("rank", -2)):
            raise ValueError(f"trainable parent adapter rank {ac.get('r')} does not match this run's LoRA rank {lc.get('rank')}")
        if float(ac.get("lora_alpha", -1.0)) != float(lc.get("alpha", -2.0)):
            raise ValueError(f"trainable parent adapter alpha {ac.get('lora_alpha')} does not match this run's LoRA alpha {lc.get('alpha')}")
        if lc.get("targets") and set(ac.get("target_modules") or ()) != set(lc["targets"]):
            raise ValueError("trainable parent adapter targets do not match this run's lora_target_modules")
    trainer.lora.load_peft(adapter_path)
    if mode in ("resume", "trainable"):
        return "resumed"
    trainer.lora.merge_into(trainer.store)
    trainer.recipe.on_weights_updated(trainer.store)
    trainer.lora.init_weights(trainer.cfg.seed + 1)  # fresh adapters: A random, B zero
    if mode == "stack" and output_dir:
        dst = os.path.join(output_dir, "previous_adapter")
        if os.path.isdir(adapter_path) and not os.path.exists(dst):
            shutil.copytree(adapter_path, dst)
    return "merged"

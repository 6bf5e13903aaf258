"""Starting a run from an existing adapter (``adapter_path`` + ``adapter_init_mode``).

* ``merge``  — fold the adapter into the base weights, then train fresh adapters on top (continual fine-tuning);
* ``resume`` — load the adapter into the trainable LoRA weights and keep training it;
* ``stack``  — like merge, but the old adapter is also kept in the output for reference.

Parity: surogate/train/adapter_init.py.
"""
from __future__ import annotations

import os
import shutil


def apply_adapter_init(trainer, adapter_path: str, mode: str = "merge", output_dir: str = "") -> str:
    if trainer.lora is None:
        raise ValueError("adapter_path needs lora: true")
    if mode not in ("merge", "resume", "stack"):
        raise ValueError(f"[E140] adapter_init_mode must be merge | resume | stack, got '{mode}'")
    trainer.lora.load_peft(adapter_path)
    if mode == "resume":
        return "resumed"
    trainer.lora.merge_into(trainer.store)
    trainer.recipe.on_weights_updated(trainer.store)
    trainer.lora.init_weights(trainer.cfg.seed + 1)  # fresh adapters: A random, B zero
    if mode == "stack" and output_dir:
        dst = os.path.join(output_dir, "previous_adapter")
        if os.path.isdir(adapter_path) and not os.path.exists(dst):
            shutil.copytree(adapter_path, dst)
    return "merged"

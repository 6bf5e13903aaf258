"""Merge a PEFT LoRA adapter into a HuggingFace checkpoint directly on safetensors files (no model is instantiated).

For every ``<module>.lora_A.weight`` / ``<module>.lora_B.weight`` pair the base tensor ``<module>.weight`` becomes
``W + scale * B @ A`` (``scale = alpha / r``, or ``alpha / sqrt(r)`` with rsLoRA); stacked expert adapters
(``...experts.<e>.<proj>``) are handled the same way because they are ordinary module paths.  Shards are processed one
at a time, so peak host memory is one shard.

Parity: surogate/utils/adapter_merge.py.
"""
from __future__ import annotations

import json
import math
import os
import shutil
from typing import Dict, Tuple

import torch
from safetensors import safe_open
from safetensors.torch import save_file


def _strip(key: str) -> str:
    for p in ("base_model.model.", "base_model."):
        if key.startswith(p):
            key = key[len(p):]
    return key


def read_adapter(adapter_dir: str) -> Tuple[Dict[str, Tuple[torch.Tensor, torch.Tensor]], float]:
    with open(os.path.join(adapter_dir, "adapter_config.json")) as f:
        cfg = json.load(f)
    r, alpha = cfg["r"], cfg["lora_alpha"]
    scale = alpha / (math.sqrt(r) if cfg.get("use_rslora") else r)
    pairs: Dict[str, Dict[str, torch.Tensor]] = {}
    with safe_open(os.path.join(adapter_dir, "adapter_model.safetensors"), framework="pt") as f:
        for k in f.keys():
            base = _strip(k)
            for tag in (".lora_A.weight", ".lora_B.weight", ".lora_A.default.weight", ".lora_B.default.weight"):
                if base.endswith(tag):
                    mod = base[: -len(tag)]
                    pairs.setdefault(mod, {})["A" if "lora_A" in tag else "B"] = f.get_tensor(k)
    out = {m + ".weight": (d["A"], d["B"]) for m, d in pairs.items() if "A" in d and "B" in d}
    return out, scale


def merge_adapter(base_dir: str, adapter_dir: str, out_dir: str, dtype: torch.dtype = torch.bfloat16) -> Dict[str, int]:
    pairs, scale = read_adapter(adapter_dir)
    os.makedirs(out_dir, exist_ok=True)
    merged, seen = 0, set()
    for fn in sorted(os.listdir(base_dir)):
        src = os.path.join(base_dir, fn)
        if fn.endswith(".safetensors"):
            tensors = {}
            with safe_open(src, framework="pt") as f:
                meta = f.metadata() or {"format": "pt"}
                for k in f.keys():
                    t = f.get_tensor(k)
                    if k in pairs:
                        A, B = pairs[k]
                        t = (t.float() + scale * (B.float() @ A.float())).to(t.dtype if t.dtype.is_floating_point else dtype)
                        merged += 1
                        seen.add(k)
                    tensors[k] = t.contiguous()
            save_file(tensors, os.path.join(out_dir, fn), metadata=meta)
        elif os.path.isfile(src):
            shutil.copy2(src, os.path.join(out_dir, fn))
    missing = sorted(set(pairs) - seen)
    if missing:
        raise KeyError(f"adapter modules without a base weight in {base_dir}: {missing[:5]}{' ...' if len(missing) > 5 else ''}")
    return {"merged": merged, "adapter_modules": len(pairs)}

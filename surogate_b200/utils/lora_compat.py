"""Compatibility fixes for adapters consumed by PEFT and vLLM.

* vLLM loads per-expert MoE adapters only under ``...mlp.experts.<e>.<proj>`` names and rejects ``modules_to_save``;
* PEFT expects ``base_model.model.`` prefixes and ``target_modules`` as a list of leaf names;
* adapters written with fused ``qkv`` / ``gate_up`` targets are split into the per-projection form both understand.

Parity: surogate/utils/lora_compat.py.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

PREFIX = "base_model.model."


def normalise_keys(tensors: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in tensors.items():
        k = k.replace(".lora_A.default.", ".lora_A.").replace(".lora_B.default.", ".lora_B.")
        if not k.startswith(PREFIX):
            k = PREFIX + (k[len("base_model."):] if k.startswith("base_model.") else k)
        out[k] = v
    return out


def split_fused(tensors: Dict[str, torch.Tensor], q_rows: int, kv_rows: int, ff_rows: int) -> Dict[str, torch.Tensor]:
    """``qkv_proj`` -> q/k/v_proj and ``gate_up_proj`` -> up/gate (rows in that storage order) by slicing lora_B rows; lora_A is shared."""
    out = dict(tensors)
    for k in list(tensors):
        if ".qkv_proj.lora_B." in k:
            B = out.pop(k)
            A = out.pop(k.replace("lora_B", "lora_A"))
            for name, lo, hi in (("q_proj", 0, q_rows), ("k_proj", q_rows, q_rows + kv_rows), ("v_proj", q_rows + kv_rows, q_rows + 2 * kv_rows)):
                out[k.replace("qkv_proj", name)] = B[lo:hi].contiguous()
                out[k.replace("qkv_proj", name).replace("lora_B", "lora_A")] = A.clone()
        elif ".gate_up_proj.lora_B." in k:
            B = out.pop(k)
            A = out.pop(k.replace("lora_B", "lora_A"))
            for name, lo, hi in (("up_proj", 0, ff_rows), ("gate_proj", ff_rows, 2 * ff_rows)):
                out[k.replace("gate_up_proj", name)] = B[lo:hi].contiguous()
                out[k.replace("gate_up_proj", name).replace("lora_B", "lora_A")] = A.clone()
    return out


def fix_adapter_config(cfg: Dict) -> Dict:
    cfg = dict(cfg)
    tm = cfg.get("target_modules")
    if isinstance(tm, str):
        tm = [tm]
    cfg["target_modules"] = sorted({t.split(".")[-1] for t in (tm or [])})
    cfg["modules_to_save"] = None
    cfg.setdefault("peft_type", "LORA")
    cfg.setdefault("task_type", "CAUSAL_LM")
    cfg.setdefault("bias", "none")
    return cfg


def make_compatible(adapter_dir: str, out_dir: str = None) -> str:
    from safetensors.torch import load_file, save_file

    out_dir = out_dir or adapter_dir
    os.makedirs(out_dir, exist_ok=True)
    t = normalise_keys(load_file(os.path.join(adapter_dir, "adapter_model.safetensors")))
    save_file(t, os.path.join(out_dir, "adapter_model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(adapter_dir, "adapter_config.json")) as f:
        cfg = fix_adapter_config(json.load(f))
    with open(os.path.join(out_dir, "adapter_config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    return out_dir

"""Derive model facts from an HF ``config.json``: architecture family, MoE / multimodal flags, dtype, pre-quantisation.

Parity: surogate/core/model/registry.py, hf_config.py (HfConfigFactory).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

MULTIMODAL_KEYS = ("vision_config", "visual", "audio_config", "image_token_id", "vision_start_token_id")
MOE_KEYS = ("num_experts", "num_local_experts", "n_routed_experts", "moe_intermediate_size")


def _text_config(cfg: Dict[str, Any]) -> Dict[str, Any]:
    return cfg.get("text_config") or cfg


def quant_info(cfg: Dict[str, Any]) -> Optional[Dict[str, Any]]:
    """Pre-quantised checkpoints: ``prequant_fp8`` (block-wise FP8), ``prequant_nvfp4`` (ModelOpt), ``prequant_mxfp4``, ``bnb_nf4``."""
    q = cfg.get("quantization_config")
    if not q:
        return None
    method = str(q.get("quant_method", "")).lower()
    if method == "fp8":
        return {"kind": "prequant_fp8", "block_size": q.get("weight_block_size"), "fmt": q.get("fmt", "e4m3")}
    if method in ("modelopt", "nvfp4") or str(q.get("quant_algo", "")).upper() == "NVFP4":
        return {"kind": "prequant_nvfp4", "group_size": q.get("group_size", 16)}
    if method == "mxfp4":
        return {"kind": "prequant_mxfp4", "modules_to_not_convert": q.get("modules_to_not_convert", [])}
    if method == "bitsandbytes" and (q.get("load_in_4bit") or q.get("bnb_4bit_quant_type")):
        return {"kind": "bnb_nf4", "double_quant": bool(q.get("bnb_4bit_use_double_quant")), "quant_type": q.get("bnb_4bit_quant_type", "nf4")}
    return {"kind": method or "unknown"}


def supported_architectures() -> List[str]:
    from ..dsl import models  # noqa: F401  (registers the model classes)
    from ..dsl.nn import registered_architectures

    return registered_architectures()


def describe_config(cfg: Dict[str, Any]) -> Dict[str, Any]:
    t = _text_config(cfg)
    arch = (cfg.get("architectures") or [cfg.get("architecture", "")])[0]
    experts = next((t[k] for k in ("num_experts", "num_local_experts", "n_routed_experts") if t.get(k)), 0)
    info = {
        "architecture": arch, "model_type": cfg.get("model_type"),
        "is_moe": bool(experts), "num_experts": int(experts or 0), "num_experts_per_tok": int(t.get("num_experts_per_tok", 0) or 0),
        "is_multimodal": any(k in cfg for k in MULTIMODAL_KEYS),
        "torch_dtype": cfg.get("torch_dtype") or cfg.get("dtype") or "bfloat16",
        "hidden_size": t.get("hidden_size"), "num_hidden_layers": t.get("num_hidden_layers"), "vocab_size": t.get("vocab_size"),
        "max_position_embeddings": t.get("max_position_embeddings"), "tie_word_embeddings": bool(cfg.get("tie_word_embeddings", t.get("tie_word_embeddings", False))),
        "quant_info": quant_info(cfg), "rope_scaling": t.get("rope_scaling"), "sliding_window": t.get("sliding_window"),
    }
    try:
        info["supported"] = arch in supported_architectures()
    except Exception:  # noqa: BLE001
        info["supported"] = None
    return info

"""HuggingFace checkpoint import / export through the mappings declared in the DSL.

Import reads ``model.safetensors`` or a sharded ``model.safetensors.index.json`` lazily (one tensor at
a time, so a 30B checkpoint never sits in host memory twice), fuses / stacks the pieces into the
internal layout ([q;k;v], [up;gate], experts on dim 0) and writes each rank's slice of the bucket.
Export is the exact inverse and produces ``config.json`` + ``model.safetensors`` with HF names.

Parity: csrc/src/runtime/dsl weight loader + utilities/safetensors.cpp; surogate/dsl/hf.py mappings.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, List, Optional

import torch
from safetensors import safe_open
from safetensors.torch import save_file

from ..dsl.compiler import CompiledModel


class LazyCheckpoint:
    """Name -> tensor access over one or many safetensors files."""

    def __init__(self, path: str, device: Optional[torch.device] = None):
        """``device``: a CUDA device makes ``get`` read tensors straight into device memory through the native reader (pinned
        double-buffered staging, or GPUDirect Storage with ``SUROGATE_GDS=1``), so fusing / stacking runs on the GPU."""
        self.device = device if (device is not None and torch.device(device).type == "cuda") else None
        self._native: Dict[str, Any] = {}
        self.dir = path if os.path.isdir(path) else os.path.dirname(path)
        self.files: Dict[str, str] = {}
        self._open: Dict[str, Any] = {}
        index = os.path.join(self.dir, "model.safetensors.index.json")
        if os.path.isfile(path) and path.endswith(".safetensors"):
            self._scan(path)
        elif os.path.exists(index):
            with open(index) as f:
                for name, fn in json.load(f)["weight_map"].items():
                    self.files[name] = os.path.join(self.dir, fn)
        else:
            single = os.path.join(self.dir, "model.safetensors")
            if not os.path.exists(single):
                raise FileNotFoundError(f"no model.safetensors or model.safetensors.index.json under {self.dir}")
            self._scan(single)

    def _scan(self, fn: str) -> None:
        with safe_open(fn, framework="pt") as f:
            for k in f.keys():
                self.files[k] = fn

    def __contains__(self, name: str) -> bool:
        return name in self.files

    def get(self, name: str) -> torch.Tensor:
        fn = self.files[name]
        if self.device is not None:
            from .safetensors_native import NativeSafetensors

            nat = self._native.get(fn)
            if nat is None:
                nat = self._native[fn] = NativeSafetensors(fn)
            return nat.get_tensor_device(name, self.device)
        h = self._open.get(fn)
        if h is None:
            h = self._open[fn] = safe_open(fn, framework="pt")
        return h.get_tensor(name)

    def names(self):
        return list(self.files)


def import_hf_weights(cm: CompiledModel, store, path: str, strict: bool = True) -> Dict[str, int]:
    direct = os.environ.get("SUROGATE_DEVICE_LOAD", "0") == "1" or os.environ.get("SUROGATE_GDS", "0") == "1"
    ckpt = LazyCheckpoint(path, device=store.device if direct else None)
    cfg_path = os.path.join(ckpt.dir, "config.json")
    hf_cfg = None
    if os.path.exists(cfg_path):
        with open(cfg_path) as f:
            hf_cfg = json.load(f)
    from .prequant import wrap_if_quantized

    ckpt = wrap_if_quantized(ckpt, hf_cfg)      # block-FP8 / NVFP4 / MXFP4 / bitsandbytes checkpoints hand out dequantised tensors
    loaded = missing = 0
    for p in cm.params:
        m = p.spec.hf
        if m is None:
            continue
        names = m.hf_names(p.layer)
        if p.tied_to:
            continue  # shares storage with its target
        if hasattr(store, "holds") and not store.holds(p.name):
            continue  # held by another pipeline stage
        if not all(n in ckpt for n in names):
            if type(m).__name__ == "tied_to":
                continue
            if strict:
                raise KeyError(f"checkpoint lacks {[n for n in names if n not in ckpt]} needed for '{p.name}'")
            missing += 1
            continue
        t = m.load(ckpt.get, p.layer)
        store.load_tensor(p.name, t)
        loaded += 1
    out = {"loaded": loaded, "missing": missing}
    if hasattr(ckpt, "stats"):
        out["dequantised"] = {k: v for k, v in ckpt.stats.items() if v and k != "plain"}
    return out


def export_hf_weights(cm: CompiledModel, store, out_dir: str, hf_config: Optional[Dict[str, Any]] = None, write: bool = True,
                      dtype: torch.dtype = torch.bfloat16, max_shard_bytes: int = 5 << 30, passthrough_from: Optional[str] = None) -> None:
    """Gather every parameter (collective when sharded), split back to HF names; rank with ``write`` saves.
    Tensors of ``passthrough_from`` (the imported checkpoint) that no parameter maps to, such as a frozen vision tower,
    are copied unchanged so the exported directory stays loadable as the full model."""
    tensors: Dict[str, torch.Tensor] = {}
    entries = {p.name: p for p in cm.params}
    for name, full in store.named_full_tensors():
        p = entries[name]
        if p.spec.hf is None:
            continue
        if write:
            # inverse mappings run at the master's precision, the cast comes last: a zero-centred norm weight stored as w - 1
            # would lose most of its bits if 1 + w were rounded to bfloat16 first
            for hf_name, t in p.spec.hf.export(full.detach().to("cpu"), p.layer).items():
                tensors[hf_name] = t.to(dtype).contiguous()
    for p in cm.params:  # untied export of tied heads keeps HF loaders happy only if the config says untied
        if p.tied_to and write and hf_config is not None and not hf_config.get("tie_word_embeddings", True):
            src = entries[p.tied_to]
            tensors[p.spec.hf.hf_names(None)[0]] = tensors[src.spec.hf.hf_names(None)[0]].clone()
    if not write:
        return
    if passthrough_from:
        try:
            src_ckpt = LazyCheckpoint(passthrough_from)
        except FileNotFoundError:
            src_ckpt = None
        if src_ckpt is not None:
            owned = {n for p in cm.params if p.spec.hf is not None for n in p.spec.hf.hf_names(p.layer)}
            for n in src_ckpt.names():
                if n not in tensors and n not in owned:
                    tensors[n] = src_ckpt.get(n).contiguous()
    os.makedirs(out_dir, exist_ok=True)
    total = sum(t.numel() * t.element_size() for t in tensors.values())
    if total <= max_shard_bytes:
        save_file(tensors, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
    else:
        shards, cur, size = [], {}, 0
        for k, t in tensors.items():
            b = t.numel() * t.element_size()
            if cur and size + b > max_shard_bytes:
                shards.append(cur)
                cur, size = {}, 0
            cur[k] = t
            size += b
        shards.append(cur)
        weight_map = {}
        for i, sh in enumerate(shards):
            fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            save_file(sh, os.path.join(out_dir, fn), metadata={"format": "pt"})
            weight_map.update({k: fn for k in sh})
        with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1)
    if hf_config is not None:
        with open(os.path.join(out_dir, "config.json"), "w") as f:
            json.dump(to_hf_config(cm, hf_config), f, indent=1)


TOKENIZER_FILES = ("tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "vocab.json", "merges.txt", "added_tokens.json", "tokenizer.model",
                   "chat_template.jinja", "chat_template.json", "generation_config.json", "preprocessor_config.json", "video_preprocessor_config.json")


def copy_tokenizer_files(src_dir: Optional[str], out_dir: str) -> List[str]:
    """Tokenizer, chat template, generation and pre-processor files of the source model next to exported weights, so the export
    loads in transformers / an inference engine without the original directory.  Files already present are kept."""
    import shutil

    copied: List[str] = []
    if not src_dir:
        return copied
    src_dir = src_dir if os.path.isdir(src_dir) else os.path.dirname(src_dir)
    if not os.path.isdir(src_dir) or os.path.abspath(src_dir) == os.path.abspath(out_dir):
        return copied
    os.makedirs(out_dir, exist_ok=True)
    for fn in TOKENIZER_FILES:
        s, d = os.path.join(src_dir, fn), os.path.join(out_dir, fn)
        if os.path.isfile(s) and not os.path.exists(d):
            shutil.copy2(s, d)
            copied.append(fn)
    return copied


def to_hf_config(cm: CompiledModel, cfg: Dict[str, Any]) -> Dict[str, Any]:
    """An HF-style config.json for the model (passes through a real HF config, derives one from ctor kwargs)."""
    if "architectures" in cfg:
        return dict(cfg)
    model = cm.model
    inv = {mine: theirs for mine, theirs in type(model).hf_config_map.items()}
    out = {"architectures": [type(model).hf_architecture], "model_type": type(model).hf_model_type, "torch_dtype": "bfloat16"}
    for mine, theirs in inv.items():
        if hasattr(model, mine):
            out[theirs] = getattr(model, mine)
    return out

"""Compile a DSL model: trace -> validate -> derive backward graphs -> parameter table.

The result (:class:`CompiledModel`) is everything the runtime needs and nothing
model-specific is left in Python callbacks: forward/backward op lists for the
model shell and for each block type, the list of tensors each backward graph
reads from its forward ("saved"), and the flat parameter table with HF mappings.

Parity: surogate/dsl/py_compiler.py (compile_model_for_hf :2282),
surogate/dsl/ir_builder.py:94 (build_dsl_ir_for_model).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .autodiff import derive_backward_graph
from .ir import Graph, ParamSpec
from .nn import Model, model_class_for


@dataclass
class ParamEntry:
    name: str  # full name, e.g. "blocks.3.qkv_weight" or "embedding"
    local: str  # name inside its graph
    spec: ParamSpec
    layer: Optional[int]  # None for model-level params
    group: str  # "embedding" | "lm_head" | "final" | "layer{L}"
    tied_to: Optional[str] = None


@dataclass
class CompiledModel:
    model: Model
    fwd: Graph
    bwd: Graph
    block_fwd: Dict[str, Graph]
    block_bwd: Dict[str, Graph]
    layer_types: List[str]
    params: List[ParamEntry] = field(default_factory=list)

    @property
    def n_layers(self) -> int:
        return len(self.layer_types)

    def param_names(self) -> List[str]:
        return [p.name for p in self.params]

    def entry(self, name: str) -> ParamEntry:
        for p in self.params:
            if p.name == name:
                return p
        raise KeyError(name)

    def num_parameters(self, unique: bool = True) -> int:
        n = 0
        for p in self.params:
            if unique and p.tied_to:
                continue
            k = 1
            for s in p.spec.shape:
                k *= s
            n += k
        return n

    def to_json(self) -> Dict[str, Any]:
        return {
            "model": type(self.model).__name__,
            "config": self.model.describe(),
            "forward": self.fwd.to_json(),
            "backward": self.bwd.to_json(),
            "blocks": {k: {"forward": g.to_json(), "backward": self.block_bwd[k].to_json()} for k, g in self.block_fwd.items()},
            "layer_types": self.layer_types,
            "params": [{"name": p.name, "layer": p.layer, "group": p.group, "tied_to": p.tied_to, **p.spec.to_json()} for p in self.params],
        }


def compile_model(model: Model, fuse: bool = True) -> CompiledModel:
    from .graph_compiler import annotate_consumers, apply_fusion_rules

    fwd = model.trace()
    fusion_report = apply_fusion_rules(fwd) if fuse else {}   # before autodiff: the backward is derived from the fused forward
    stack_ops = [op for op in fwd.ops if op.kind == "block_stack"]
    layer_types: List[str] = []
    block_fwd: Dict[str, Graph] = {}
    block_bwd: Dict[str, Graph] = {}
    if stack_ops:
        if len(stack_ops) != 1:
            raise ValueError("[E021] a model may contain exactly one block stack")
        layer_types = list(stack_ops[0].attrs["layer_types"])
        for name, g in fwd.subgraphs.items():
            block_fwd[name] = g
            block_bwd[name] = derive_backward_graph(g, wrt_inputs=["x", "residual"])
            annotate_consumers(g)
            annotate_consumers(block_bwd[name])
    bwd = derive_backward_graph(fwd)
    fwd.meta["fusion_report"] = fusion_report

    params: List[ParamEntry] = []
    for name, spec in fwd.params.items():
        if name == "embedding":
            group = "embedding"
        elif name == "lm_head":
            group = "lm_head"
        else:
            group = "final"
        tied = getattr(spec.hf, "other", None) if spec.hf is not None and type(spec.hf).__name__ == "tied_to" else None
        params.append(ParamEntry(name, name, spec, None, group, tied))
    for L, bt in enumerate(layer_types):
        for local, spec in block_fwd[bt].params.items():
            params.append(ParamEntry(f"blocks.{L}.{local}", local, spec, L, f"layer{L}"))
    # embedding first, blocks, then final norm / lm head: the order weights are needed in forward
    order = {"embedding": 0, "final": 2, "lm_head": 3}
    params.sort(key=lambda p: (1, p.layer) if p.layer is not None else (order[p.group], 0))
    return CompiledModel(model, fwd, bwd, block_fwd, block_bwd, layer_types, params)


def load_hf_config(model_dir_or_cfg) -> Dict[str, Any]:
    if isinstance(model_dir_or_cfg, dict):
        return dict(model_dir_or_cfg)
    path = model_dir_or_cfg
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    with open(path) as f:
        return json.load(f)


def model_from_hf_config(cfg: Dict[str, Any], **overrides) -> Model:
    arch = (cfg.get("architectures") or [cfg.get("model_type")])[0]
    try:
        cls = model_class_for(arch)
    except KeyError:
        cls = model_class_for(cfg.get("model_type", arch))
    return cls.from_hf_config(cfg, **overrides)


def build_dsl_ir_for_model(model_dir_or_cfg, extra_config: Optional[Dict[str, Any]] = None) -> str:
    """Trace the model described by an HF ``config.json`` (path, directory or dict) and return its IR as JSON."""
    cfg = load_hf_config(model_dir_or_cfg)
    model = model_from_hf_config(cfg, **(extra_config or {}))
    return json.dumps(compile_model(model).to_json(), default=str)

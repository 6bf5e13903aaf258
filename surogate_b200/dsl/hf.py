"""HF checkpoint <-> internal parameter mappings, declared next to the parameters.

Internal layouts are fused ([q;k;v] rows, [up;gate] rows, experts stacked on
dim 0); HF checkpoints store the pieces separately.  A mapping object knows how
to *load* (gather HF tensors into one internal tensor) and how to *export*
(split the internal tensor back into HF tensors), so import and export stay
exact inverses.  ``{L}`` in a template is the layer index, ``{E}`` the expert.

Parity: surogate/dsl/hf.py (fuse :136, split :157, transform :193, tied_to :207,
stack_experts :220, build_dense_block_mappings :526).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch


class Mapping:
    def hf_names(self, layer: Optional[int]) -> List[str]:
        raise NotImplementedError

    def load(self, get: Callable[[str], torch.Tensor], layer: Optional[int]) -> torch.Tensor:
        raise NotImplementedError

    def export(self, tensor: torch.Tensor, layer: Optional[int]) -> Dict[str, torch.Tensor]:
        raise NotImplementedError

    def to_json(self):
        return {"kind": type(self).__name__, **{k: v for k, v in vars(self).items() if not callable(v)}}


def _fmt(t: str, layer: Optional[int], expert: Optional[int] = None) -> str:
    if layer is not None:
        t = t.replace("{L}", str(layer))
    if expert is not None:
        t = t.replace("{E}", str(expert))
    return t


@dataclass
class direct(Mapping):
    template: str

    def hf_names(self, layer):
        return [_fmt(self.template, layer)]

    def load(self, get, layer):
        return get(_fmt(self.template, layer))

    def export(self, tensor, layer):
        return {_fmt(self.template, layer): tensor}


@dataclass
class fuse(Mapping):
    """Concatenate several HF tensors along ``dim`` (rows by default) in the given order."""
    templates: Sequence[str]
    dim: int = 0
    sizes: Optional[Sequence[int]] = None  # sizes along dim for export (filled at load or by the module)

    def hf_names(self, layer):
        return [_fmt(t, layer) for t in self.templates]

    def load(self, get, layer):
        parts = [get(n) for n in self.hf_names(layer)]
        if self.sizes is None:
            self.sizes = [p.shape[self.dim] for p in parts]
        return torch.cat(parts, dim=self.dim)

    def export(self, tensor, layer):
        assert self.sizes is not None, "fuse mapping needs sizes to export"
        parts = torch.split(tensor, list(self.sizes), dim=self.dim)
        return {n: p.contiguous() for n, p in zip(self.hf_names(layer), parts)}


@dataclass
class transform(Mapping):
    """Apply an invertible function on load (and its inverse on export)."""
    template: str
    fn: str = "identity"  # identity | transpose | plus_one (gemma-style norm offsets) | swap_row_halves ([gate; up] <-> [up; gate])

    def hf_names(self, layer):
        return [_fmt(self.template, layer)]

    def _apply(self, t, inverse):
        if self.fn == "transpose":
            return t.transpose(-1, -2).contiguous()
        if self.fn == "plus_one":
            return t - 1 if inverse else t + 1
        if self.fn == "swap_row_halves":  # its own inverse
            a, b = t.chunk(2, dim=-2)
            return torch.cat([b, a], dim=-2).contiguous()
        return t

    def load(self, get, layer):
        return self._apply(get(_fmt(self.template, layer)), False)

    def export(self, tensor, layer):
        return {_fmt(self.template, layer): self._apply(tensor, True)}


@dataclass
class tied_to(Mapping):
    """Parameter shares storage with ``other`` when the checkpoint has no tensor of its own."""
    template: str
    other: str

    def hf_names(self, layer):
        return [_fmt(self.template, layer)]

    def load(self, get, layer):
        return get(_fmt(self.template, layer))

    def export(self, tensor, layer):
        return {_fmt(self.template, layer): tensor}


@dataclass
class stack_experts(Mapping):
    """Stack per-expert HF tensors on a new dim 0; optionally fuse two projections per expert on rows."""
    templates: Sequence[str]  # one template (plain) or several (fused along rows, in order)
    num_experts: int = 0
    sizes: Optional[Sequence[int]] = None

    def hf_names(self, layer):
        return [_fmt(t, layer, e) for e in range(self.num_experts) for t in self.templates]

    def load(self, get, layer):
        rows = []
        for e in range(self.num_experts):
            parts = [get(_fmt(t, layer, e)) for t in self.templates]
            if self.sizes is None:
                self.sizes = [p.shape[0] for p in parts]
            rows.append(torch.cat(parts, dim=0) if len(parts) > 1 else parts[0])
        return torch.stack(rows, dim=0)

    def export(self, tensor, layer):
        out = {}
        for e in range(tensor.shape[0]):
            if len(self.templates) == 1:
                out[_fmt(self.templates[0], layer, e)] = tensor[e].contiguous()
            else:
                parts = torch.split(tensor[e], list(self.sizes), dim=0)
                for t, p in zip(self.templates, parts):
                    out[_fmt(t, layer, e)] = p.contiguous()
        return out


def build_dense_block_mappings(prefix: str = "model.layers.{L}") -> Dict[str, Mapping]:
    """Standard Llama/Qwen-family block: canonical internal name -> HF mapping."""
    a, m = f"{prefix}.self_attn", f"{prefix}.mlp"
    return {
        "ln1_weight": direct(f"{prefix}.input_layernorm.weight"),
        "ln2_weight": direct(f"{prefix}.post_attention_layernorm.weight"),
        "qkv_weight": fuse([f"{a}.q_proj.weight", f"{a}.k_proj.weight", f"{a}.v_proj.weight"]),
        "qkv_bias": fuse([f"{a}.q_proj.bias", f"{a}.k_proj.bias", f"{a}.v_proj.bias"]),
        "out_weight": direct(f"{a}.o_proj.weight"),
        "q_norm_weight": direct(f"{a}.q_norm.weight"),
        "k_norm_weight": direct(f"{a}.k_norm.weight"),
        "mlp_up_weight": fuse([f"{m}.up_proj.weight", f"{m}.gate_proj.weight"]),
        "mlp_down_weight": direct(f"{m}.down_proj.weight"),
    }


def build_moe_block_mappings(num_experts: int, prefix: str = "model.layers.{L}") -> Dict[str, Mapping]:
    a, m = f"{prefix}.self_attn", f"{prefix}.mlp"
    d = build_dense_block_mappings(prefix)
    del d["mlp_up_weight"], d["mlp_down_weight"]
    d.update({
        "router_weight": direct(f"{m}.gate.weight"),
        "experts_gate_up": stack_experts([f"{m}.experts.{{E}}.up_proj.weight", f"{m}.experts.{{E}}.gate_proj.weight"], num_experts),
        "experts_down": stack_experts([f"{m}.experts.{{E}}.down_proj.weight"], num_experts),
    })
    return d


#: LoRA target name -> (internal param, piece index within the fused rows) for PEFT export
LORA_TARGETS = {
    "q_proj": ("qkv_weight", 0), "k_proj": ("qkv_weight", 1), "v_proj": ("qkv_weight", 2), "o_proj": ("out_weight", 0),
    "up_proj": ("mlp_up_weight", 0), "gate_proj": ("mlp_up_weight", 1), "down_proj": ("mlp_down_weight", 0),
}

"""Laguna (``LagunaForCausalLM``): per-layer choice of full / sliding-window attention (different rotary base, rotary fraction,
scaling and query-head count per kind) and of dense / sparse feed-forward; untied LM head.

Parity: surogate/dsl/models/laguna.py.
"""
from __future__ import annotations

from typing import Dict, List, Optional

from .. import functional as F
from .. import nn
from ..blocks import STANDARD_MODEL_NAME_REMAP
from ..blocks.laguna import LagunaDenseBlock, LagunaSparseBlock
from ..modules import Embedding, LMHead, RMSNorm


def layer_structure(n_layers: int, layer_types, mlp_layer_types, heads_per_layer, num_query_heads: int):
    """Per-layer block kind ("full_dense", "sliding_sparse", ...) and the query-head count of each attention kind (which must
    be uniform within a kind: one traced block serves all its layers)."""
    layer_types = list(layer_types or ["full_attention"] * n_layers)
    mlp_layer_types = list(mlp_layer_types or (["dense"] + ["sparse"] * (n_layers - 1)))
    heads_per_layer = list(heads_per_layer or [num_query_heads] * n_layers)
    for name, v in (("layer_types", layer_types), ("mlp_layer_types", mlp_layer_types), ("num_attention_heads_per_layer", heads_per_layer)):
        if len(v) != n_layers:
            raise ValueError(f"{name} has {len(v)} entries for {n_layers} layers")
    kinds: List[str] = []
    heads: Dict[str, int] = {}
    for lt, mt, h in zip(layer_types, mlp_layer_types, heads_per_layer):
        attn = {"full_attention": "full", "sliding_attention": "sliding"}.get(lt)
        if attn is None or mt not in ("dense", "sparse"):
            raise ValueError(f"unknown layer kind ({lt}, {mt})")
        if heads.setdefault(attn, int(h)) != int(h):
            raise ValueError(f"{lt} layers have different query-head counts ({heads[attn]} and {h})")
        kinds.append(f"{attn}_{mt}")
    return kinds, heads


@nn.hf_config(architecture="LagunaForCausalLM", model_type="laguna", d_model="hidden_size", n_layers="num_hidden_layers", num_query_heads="num_attention_heads",
              num_kv_heads="num_key_value_heads", moe_d_ff="moe_intermediate_size", d_ff="intermediate_size", vocab_size="vocab_size",
              max_seq="max_position_embeddings", head_size="head_dim", eps="rms_norm_eps", num_experts="num_experts", num_experts_per_tok="num_experts_per_tok",
              shared_d_ff="shared_expert_intermediate_size", routed_scaling_factor="moe_routed_scaling_factor",
              router_logit_softcapping="moe_router_logit_softcapping", apply_router_weight_on_input="moe_apply_router_weight_on_input", gating="gating",
              sliding_window="sliding_window", layer_types="layer_types", mlp_layer_types="mlp_layer_types",
              num_attention_heads_per_layer="num_attention_heads_per_layer", tie_word_embeddings="tie_word_embeddings", rope_parameters="rope_parameters")
class LagunaModel(nn.Model):
    _name_remap_ = STANDARD_MODEL_NAME_REMAP

    def __init__(self, vocab_size: int = 100352, d_model: int = 2048, n_layers: int = 40, num_query_heads: int = 48, num_kv_heads: int = 8, head_size: int = 128,
                 d_ff: int = 8192, moe_d_ff: int = 512, max_seq: int = 131072, eps: float = 1e-6, num_experts: int = 256, num_experts_per_tok: int = 8,
                 shared_d_ff: int = 512, routed_scaling_factor: float = 1.0, router_logit_softcapping: float = 0.0, apply_router_weight_on_input: bool = False,
                 gating=True, sliding_window: Optional[int] = 512, layer_types=None, mlp_layer_types=None, num_attention_heads_per_layer=None,
                 tie_word_embeddings: bool = False, rope_parameters=None, ep_size: int = 1):
        super().__init__()
        if router_logit_softcapping:
            raise ValueError("Laguna: moe_router_logit_softcapping != 0 is not supported")
        if apply_router_weight_on_input:
            raise ValueError("Laguna: moe_apply_router_weight_on_input is not supported")
        if tie_word_embeddings:
            raise ValueError("Laguna: tied word embeddings are not supported")
        self.vocab_size, self.d_model, self.n_layers, self.num_experts, self.ep_size = vocab_size, d_model, n_layers, num_experts, ep_size
        gate_per_head = gating is True or (isinstance(gating, str) and gating.lower() in ("per_head", "per-head", "head", "true"))
        kinds, heads = layer_structure(n_layers, layer_types, mlp_layer_types, num_attention_heads_per_layer, num_query_heads)
        rp = rope_parameters or {}
        per_kind = {"full": rp.get("full_attention") or ({} if "sliding_attention" in rp else rp), "sliding": rp.get("sliding_attention") or {}}
        classes = {}
        for kind in dict.fromkeys(kinds):
            attn, mlp = kind.split("_")
            r = dict(per_kind[attn])
            rotary_dim = int(head_size * float(r.get("partial_rotary_factor", 1.0)))
            scaling = {k: v for k, v in r.items() if k not in ("rope_theta", "partial_rotary_factor")} if (r.get("rope_type") or "default") != "default" else None
            common = dict(d_model=d_model, num_query_heads=heads[attn], num_kv_heads=num_kv_heads, head_size=head_size, max_seq=max_seq,
                          sliding_window=sliding_window if attn == "sliding" else 0, rope_theta=float(r.get("rope_theta", 10000.0)), rotary_dim=rotary_dim,
                          rope_scaling=scaling, gate_per_head=gate_per_head, eps=eps)
            if mlp == "dense":
                classes[kind] = (LagunaDenseBlock, dict(common, d_ff=d_ff))
            else:
                classes[kind] = (LagunaSparseBlock, dict(common, moe_d_ff=moe_d_ff, num_experts=num_experts, num_experts_per_tok=num_experts_per_tok,
                                                         shared_d_ff=shared_d_ff, routed_scaling_factor=routed_scaling_factor, ep_size=ep_size))
        self.embedding = Embedding(vocab_size, d_model)
        self.blocks = nn.HybridBlockStack(kinds, classes)
        self.final_norm = RMSNorm(d_model, eps=eps, hf_name="model.norm.weight")
        self.lm_head = LMHead(vocab_size, d_model)

    def forward(self, token_ids, position_ids, targets):
        x = self.embedding(token_ids)
        residual = F.zeros(("B", "T", self.d_model), name="residual0")
        x, residual = self.blocks(x, residual, position_ids)
        residual, x = self.final_norm(residual, x)
        return self.lm_head(x, targets)

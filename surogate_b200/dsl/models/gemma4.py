"""Gemma4 text model (``Gemma4ForCausalLM``; also the text decoder of ``Gemma4ForConditionalGeneration`` checkpoints).

Sliding and full attention layers alternate (``layer_types``), each kind with its own head size, key/value head count and rotary
setup; embeddings are scaled by sqrt(hidden) rounded to bfloat16 as the checkpoint's buffer is; logits can be soft-capped.
The small checkpoints add per-layer input embeddings (a second token embedding of width layers x P, mixed with a projection of
the main embedding and fed to every layer through a gated bottleneck) and let the last ``num_kv_shared_layers`` layers reuse
the keys / values of the last earlier layer of the same attention kind (optionally with a double-width feed-forward).

Parity: surogate/dsl/models/gemma4.py.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import functional as F
from .. import nn
from ..blocks import STANDARD_MODEL_NAME_REMAP
from ..blocks.gemma4 import Gemma4Block
from ..modules import Embedding, LMHead, RMSNorm


def default_layer_types(n_layers: int, pattern: int = 6) -> List[str]:
    types = ["sliding_attention" if (i + 1) % pattern else "full_attention" for i in range(n_layers)]
    types[-1] = "full_attention"  # the last layer always attends globally
    return types


@nn.hf_config(architecture="Gemma4ForCausalLM", model_type="gemma4_text", d_model="hidden_size", n_layers="num_hidden_layers", num_query_heads="num_attention_heads",
              num_kv_heads="num_key_value_heads", head_size="head_dim", global_head_size="global_head_dim", num_global_kv_heads="num_global_key_value_heads",
              d_ff="intermediate_size", vocab_size="vocab_size", max_seq="max_position_embeddings", eps="rms_norm_eps", sliding_window="sliding_window",
              layer_types="layer_types", rope_parameters="rope_parameters", final_logit_softcapping="final_logit_softcapping", k_eq_v="attention_k_eq_v",
              d_per_layer_input="hidden_size_per_layer_input", vocab_size_per_layer_input="vocab_size_per_layer_input",
              num_kv_shared_layers="num_kv_shared_layers", use_double_wide_mlp="use_double_wide_mlp", enable_moe_block="enable_moe_block",
              num_experts="num_experts", top_k_experts="top_k_experts", moe_d_ff="moe_intermediate_size", tie_word_embeddings="tie_word_embeddings")
class Gemma4Model(nn.Model):
    _name_remap_ = STANDARD_MODEL_NAME_REMAP

    def __init__(self, vocab_size: int = 262144, d_model: int = 2304, n_layers: int = 30, num_query_heads: int = 8, num_kv_heads: int = 4, head_size: int = 256,
                 global_head_size: Optional[int] = 512, num_global_kv_heads: Optional[int] = None, d_ff: int = 9216, max_seq: int = 131072, eps: float = 1e-6,
                 sliding_window: int = 512, layer_types: Optional[List[str]] = None, rope_parameters=None, final_logit_softcapping: Optional[float] = None,
                 k_eq_v: bool = False, d_per_layer_input: int = 0, vocab_size_per_layer_input: Optional[int] = None, num_kv_shared_layers: int = 0,
                 use_double_wide_mlp: bool = False, enable_moe_block: bool = False, num_experts: Optional[int] = None,
                 top_k_experts: Optional[int] = None, moe_d_ff: Optional[int] = None, tie_word_embeddings: bool = True, ep_size: int = 1):
        super().__init__()
        self.d_pli = int(d_per_layer_input or 0)
        self.vocab_size, self.d_model, self.n_layers, self.ep_size = vocab_size, d_model, n_layers, ep_size
        self.num_experts = int(num_experts or 0)
        types = list(layer_types) if layer_types else default_layer_types(n_layers)
        rp = rope_parameters or {"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                                 "full_attention": {"rope_type": "proportional", "rope_theta": 1000000.0, "partial_rotary_factor": 0.25}}
        moe = dict(moe=True, moe_d_ff=int(moe_d_ff or 0), num_experts=self.num_experts, top_k=int(top_k_experts or 0), ep_size=ep_size) if enable_moe_block else {}
        # layer roles for key / value sharing: the last ``num_kv_shared_layers`` layers borrow from the last earlier layer of their kind
        first_shared = n_layers - int(num_kv_shared_layers or 0) if num_kv_shared_layers else n_layers
        roles = [""] * n_layers
        for i in range(first_shared, n_layers):
            roles[i] = "shared"
            producer = max(j for j in range(first_shared) if types[j] == types[i])
            roles[producer] = "producer"
        kinds = [t + (":" + r if r else "") for t, r in zip(types, roles)]
        classes = {}
        for kind in dict.fromkeys(kinds):
            base, _, role = kind.partition(":")
            full = base == "full_attention"
            r = dict(rp.get(base) or {})
            scaling = {k: v for k, v in r.items() if k != "rope_theta"} if (r.get("rope_type") or "default") != "default" else None
            alt = bool(k_eq_v) and full
            classes[kind] = (Gemma4Block, dict(d_model=d_model, num_query_heads=num_query_heads, num_kv_heads=(num_global_kv_heads or num_kv_heads) if alt else num_kv_heads,
                                               head_size=(global_head_size or head_size) if full else head_size,
                                               d_ff=d_ff * (2 if (use_double_wide_mlp and role == "shared") else 1), window=0 if full else sliding_window,
                                               rope_theta=float(r.get("rope_theta", 10000.0)), rope_scaling=scaling, k_eq_v=alt, eps=eps, kv_role=role,
                                               kv_key="kv_" + base, d_pli=self.d_pli, **moe))
        types = kinds
        if self.d_pli:
            from .. import hf as hfmap

            vp = int(vocab_size_per_layer_input or vocab_size)
            self.declare_param("pli_embedding", (vp, n_layers * self.d_pli), decay=False, hf=hfmap.direct("model.embed_tokens_per_layer.weight"))
            self.declare_param("pli_model_proj", (n_layers * self.d_pli, d_model), hf=hfmap.direct("model.per_layer_model_projection.weight"))
            self.declare_param("pli_proj_norm", (self.d_pli,), init="ones", decay=False, hf=hfmap.direct("model.per_layer_projection_norm.weight"))
        self.eps = eps
        # the checkpoint keeps the embedding scale as a bfloat16 buffer: sqrt(3072) = 55.43 becomes 55.5
        self.embed_scale = float(torch.tensor(d_model ** 0.5).to(torch.bfloat16))
        self.embedding = Embedding(vocab_size, d_model)
        self.blocks = nn.HybridBlockStack(types, classes)
        self.final_norm = RMSNorm(d_model, eps=eps, hf_name="model.norm.weight")
        self.lm_head = LMHead(vocab_size, d_model, tie_to="embedding" if tie_word_embeddings else None, softcap=float(final_logit_softcapping or 0.0))

    def forward(self, token_ids, position_ids, targets):
        x = F.scale(self.embedding(token_ids), self.embed_scale, name="x0_scaled")
        if self.d_pli:  # computed once here, read by every layer (and differentiated back) through the shared-value channel
            x, _ = F.torch_fn("gemma4_pli", [x, token_ids, self.p("pli_embedding"), self.p("pli_model_proj"), self.p("pli_proj_norm")],
                              [("x0_pli", x.shape, "act"), ("per_layer_inputs", ("B", "T", self.n_layers, self.d_pli), "act")],
                              n_layers=self.n_layers, d_pli=self.d_pli, eps=self.eps, shared_out=[["pli", 1]])
        residual = F.zeros(("B", "T", self.d_model), name="residual0")
        x, residual = self.blocks(x, residual, position_ids)
        residual, x = self.final_norm(residual, x)
        return self.lm_head(x, targets)

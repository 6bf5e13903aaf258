"""Qwen3.5-MoE text model (``Qwen3_5MoeForCausalLM``): the Qwen3.5 hybrid of Gated DeltaNet and output-gated attention layers,
each followed by routed experts (softmax top-k, renormalised) and a sigmoid-gated shared expert.

Parity: surogate/dsl/models/qwen3_5_moe.py.
"""
from __future__ import annotations

from typing import List, Optional

from .. import functional as F
from .. import nn
from ..blocks import STANDARD_MODEL_NAME_REMAP
from ..blocks.qwen3_5 import Qwen35MoEAttentionBlock, Qwen35MoELinearBlock
from ..modules import Embedding, LMHead, RMSNorm


@nn.hf_config(architecture="Qwen3_5MoeForCausalLM", model_type="qwen3_5_moe_text", d_model="hidden_size", n_layers="num_hidden_layers",
              num_query_heads="num_attention_heads", num_kv_heads="num_key_value_heads", head_size="head_dim", moe_d_ff="moe_intermediate_size",
              shared_d_ff="shared_expert_intermediate_size", num_experts="num_experts", num_experts_per_tok="num_experts_per_tok",
              aux_loss_coef="router_aux_loss_coef", vocab_size="vocab_size", eps="rms_norm_eps", rope_theta="rope_theta", layer_types="layer_types",
              rope_parameters="rope_parameters", partial_rotary_factor="partial_rotary_factor", linear_num_key_heads="linear_num_key_heads",
              linear_num_value_heads="linear_num_value_heads", linear_key_head_dim="linear_key_head_dim", linear_value_head_dim="linear_value_head_dim",
              linear_conv_kernel_dim="linear_conv_kernel_dim", tie_word_embeddings="tie_word_embeddings")
class Qwen35MoEModel(nn.Model):
    _name_remap_ = STANDARD_MODEL_NAME_REMAP

    def __init__(self, vocab_size: int = 248320, d_model: int = 2048, n_layers: int = 40, num_query_heads: int = 16, num_kv_heads: int = 2, head_size: int = 256,
                 moe_d_ff: int = 512, shared_d_ff: int = 512, num_experts: int = 256, num_experts_per_tok: int = 8, aux_loss_coef: float = 1e-3,
                 eps: float = 1e-6, rope_theta: float = 1e7, layer_types: Optional[List[str]] = None, rope_parameters=None, partial_rotary_factor: float = 0.25,
                 linear_num_key_heads: int = 16, linear_num_value_heads: int = 32, linear_key_head_dim: int = 128, linear_value_head_dim: int = 128,
                 linear_conv_kernel_dim: int = 4, tie_word_embeddings: bool = False, ep_size: int = 1):
        super().__init__()
        self.vocab_size, self.d_model, self.n_layers, self.num_experts, self.ep_size = vocab_size, d_model, n_layers, num_experts, ep_size
        if isinstance(rope_parameters, dict):
            partial_rotary_factor = rope_parameters.get("partial_rotary_factor", partial_rotary_factor)
        types = list(layer_types) if layer_types else [("full_attention" if (i + 1) % 4 == 0 else "linear_attention") for i in range(n_layers)]
        common = dict(d_model=d_model, moe_d_ff=moe_d_ff, shared_d_ff=shared_d_ff, num_experts=num_experts, num_experts_per_tok=num_experts_per_tok,
                      norm_topk_prob=True, ep_size=ep_size, aux_loss_coef=aux_loss_coef, eps=eps)
        classes = {}
        if "full_attention" in types:
            classes["full_attention"] = (Qwen35MoEAttentionBlock, dict(common, num_query_heads=num_query_heads, num_kv_heads=num_kv_heads, head_size=head_size,
                                                                        rope_theta=float(rope_theta), rotary_dim=int(head_size * partial_rotary_factor)))
        if "linear_attention" in types:
            classes["linear_attention"] = (Qwen35MoELinearBlock, dict(common, num_k_heads=linear_num_key_heads, num_v_heads=linear_num_value_heads,
                                                                       head_k_dim=linear_key_head_dim, head_v_dim=linear_value_head_dim,
                                                                       conv_kernel=linear_conv_kernel_dim))
        self.embedding = Embedding(vocab_size, d_model, hf_name="model.language_model.embed_tokens.weight")
        self.blocks = nn.HybridBlockStack(types, classes)
        self.final_norm = RMSNorm(d_model, eps=eps, hf_name="model.language_model.norm.weight", zero_centered=True)
        self.lm_head = LMHead(vocab_size, d_model, tie_to="embedding" if tie_word_embeddings else None)

    def forward(self, token_ids, position_ids, targets):
        x = self.embedding(token_ids)
        residual = F.zeros(("B", "T", self.d_model), name="residual0")
        x, residual, aux = self.blocks(x, residual, position_ids)
        residual, x = self.final_norm(residual, x)
        return self.lm_head(x, targets), aux[0]

"""Qwen3-MoE (e.g. Qwen3-30B-A3B): every layer routes tokens to top-k of E SwiGLU experts.

Parity: surogate/dsl/models/qwen3_moe.py:31.
"""
from __future__ import annotations

from .. import functional as F
from .. import nn
from ..blocks import Qwen3MoEBlock, STANDARD_MODEL_NAME_REMAP
from ..modules import Embedding, LMHead, RMSNorm


@nn.hf_config(architecture="Qwen3MoeForCausalLM", model_type="qwen3_moe", d_model="hidden_size", n_layers="num_hidden_layers",
              num_query_heads="num_attention_heads", num_kv_heads="num_key_value_heads", moe_d_ff="moe_intermediate_size",
              vocab_size="vocab_size", max_seq="max_position_embeddings", head_size="head_dim", eps="rms_norm_eps",
              rope_theta="rope_theta", num_experts="num_experts", num_experts_per_tok="num_experts_per_tok",
              norm_topk_prob="norm_topk_prob", aux_loss_coef="router_aux_loss_coef", tie_word_embeddings="tie_word_embeddings")
class Qwen3MoEModel(nn.Model):
    _name_remap_ = STANDARD_MODEL_NAME_REMAP

    def __init__(self, vocab_size: int = 151936, d_model: int = 2048, n_layers: int = 48, num_query_heads: int = 32,
                 num_kv_heads: int = 4, moe_d_ff: int = 768, max_seq: int = 40960, head_size: int = 128, eps: float = 1e-6,
                 rope_theta: float = 1e6, num_experts: int = 128, num_experts_per_tok: int = 8, norm_topk_prob: bool = True,
                 aux_loss_coef: float = 1e-3, z_loss_coef: float = 0.0, ep_size: int = 1, shared_expert_d_ff: int = 0,
                 tie_word_embeddings: bool = False):
        super().__init__()
        self.vocab_size, self.d_model, self.n_layers = vocab_size, d_model, n_layers
        self.num_query_heads, self.num_kv_heads, self.moe_d_ff = num_query_heads, num_kv_heads, moe_d_ff
        self.head_size = head_size if head_size and head_size > 0 else d_model // num_query_heads
        self.num_experts, self.num_experts_per_tok, self.ep_size = num_experts, num_experts_per_tok, ep_size
        self.eps, self.rope_theta, self.tie_word_embeddings = eps, float(rope_theta), bool(tie_word_embeddings)
        self.embedding = Embedding(vocab_size, d_model)
        self.blocks = nn.BlockStack(
            n_layers, Qwen3MoEBlock, d_model=d_model, num_query_heads=num_query_heads, num_kv_heads=num_kv_heads,
            head_size=self.head_size, moe_d_ff=moe_d_ff, num_experts=num_experts, num_experts_per_tok=num_experts_per_tok,
            norm_topk_prob=norm_topk_prob, ep_size=ep_size, aux_loss_coef=aux_loss_coef, z_loss_coef=z_loss_coef,
            shared_expert_d_ff=shared_expert_d_ff, eps=eps, rope_theta=self.rope_theta, max_seq=max_seq)
        self.final_norm = RMSNorm(d_model, eps=eps, hf_name="model.norm.weight")
        self.lm_head = LMHead(vocab_size, d_model, tie_to="embedding" if self.tie_word_embeddings else None)

    def forward(self, token_ids, position_ids, targets):
        x = self.embedding(token_ids)
        residual = F.zeros(("B", "T", self.d_model), name="residual0")
        x, residual, aux = self.blocks(x, residual, position_ids)
        residual, x = self.final_norm(residual, x)
        loss = self.lm_head(x, targets)
        return loss, aux[0]

"""Qwen3-MoE block: QK-norm GQA attention + routed experts (optional shared expert).

Returns (moe_out, residual, aux_loss); the block stack sums aux losses over layers.

Parity: surogate/dsl/blocks/qwen3_moe.py:13.
"""
from __future__ import annotations

from .. import functional as F
from ..modules import AttentionConfig, GenericGQAttention, MoEExpertsGated, MoESharedExpert, RMSNorm
from ..nn import Block
from .common import MOE_BLOCK_NAME_REMAP

_P = "model.layers.{L}"


class Qwen3MoEBlock(Block):
    _name_remap_ = MOE_BLOCK_NAME_REMAP

    def __init__(self, d_model: int, num_query_heads: int, num_kv_heads: int, head_size: int, moe_d_ff: int, num_experts: int,
                 num_experts_per_tok: int = 8, norm_topk_prob: bool = True, ep_size: int = 1, aux_loss_coef: float = 1e-3,
                 z_loss_coef: float = 0.0, shared_expert_d_ff: int = 0, eps: float = 1e-6, rope_theta: float = 1e6,
                 use_qk_norm: bool = True, max_seq: int = 0):
        super().__init__()
        self.attn_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.input_layernorm.weight")
        self.self_attn = GenericGQAttention(d_model, num_query_heads, num_kv_heads, head_size, max_seq,
                                            config=AttentionConfig(qk_norm=use_qk_norm, eps=eps, rope_theta=rope_theta))
        self.mlp_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.post_attention_layernorm.weight")
        self.mlp = MoEExpertsGated(d_model, moe_d_ff, num_experts, num_experts_per_tok, norm_topk_prob, ep_size,
                                   aux_loss_coef, z_loss_coef)
        self.has_shared = shared_expert_d_ff > 0
        if self.has_shared:
            self.shared_expert = MoESharedExpert(d_model, shared_expert_d_ff)

    def forward(self, x, residual, position_ids):
        residual, h = self.attn_norm(residual, x)
        h = self.self_attn(h, position_ids)
        residual, h = self.mlp_norm(residual, h)
        y, aux = self.mlp(h)
        if self.has_shared:
            y = F.add(y, self.shared_expert(h), name="moe_plus_shared")
        return y, residual, aux

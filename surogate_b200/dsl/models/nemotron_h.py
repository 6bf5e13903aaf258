"""Nemotron-H (``NemotronHForCausalLM``): Mamba-2, attention and MoE mixers interleaved per ``layers_block_type``.

Parity: surogate/dsl/models/nemotron_h.py.
"""
from __future__ import annotations

from typing import List, Optional

from .. import functional as F
from .. import nn
from ..blocks.nemotron_h import NemotronHAttentionBlock, NemotronHMambaBlock, NemotronHMoEBlock
from ..modules import Embedding, LMHead, RMSNorm

_REMAP = {"embedding.weight": "embedding", "embedding.x0": "x0", "final_norm.weight": "final_norm", "final_norm.ln": "xF", "final_norm.ln_rstd": "ln_final_rstd",
          "final_norm.res": "residual_final", "lm_head.weight": "lm_head", "lm_head.loss": "loss", "blocks.*": ""}


@nn.hf_config(architecture="NemotronHForCausalLM", model_type="nemotron_h", d_model="hidden_size", layer_types="layers_block_type",
              num_query_heads="num_attention_heads", num_kv_heads="num_key_value_heads", head_size="head_dim", vocab_size="vocab_size",
              eps="layer_norm_epsilon", mamba_num_heads="mamba_num_heads", mamba_head_dim="mamba_head_dim", n_groups="n_groups",
              ssm_state_size="ssm_state_size", conv_kernel="conv_kernel", chunk_size="chunk_size", num_experts="n_routed_experts",
              num_experts_per_tok="num_experts_per_tok", moe_d_ff="moe_intermediate_size", shared_d_ff="moe_shared_expert_intermediate_size",
              n_group="n_group", topk_group="topk_group", norm_topk_prob="norm_topk_prob", routed_scaling_factor="routed_scaling_factor",
              tie_word_embeddings="tie_word_embeddings")
class NemotronHModel(nn.Model):
    _name_remap_ = _REMAP

    def __init__(self, vocab_size: int = 131072, d_model: int = 4096, layer_types: Optional[List[str]] = None, num_query_heads: int = 32, num_kv_heads: int = 8,
                 head_size: int = 128, eps: float = 1e-5, mamba_num_heads: int = 128, mamba_head_dim: int = 64, n_groups: int = 8, ssm_state_size: int = 128,
                 conv_kernel: int = 4, chunk_size: int = 128, num_experts: int = 8, num_experts_per_tok: int = 2, moe_d_ff: int = 7688, shared_d_ff: int = 7688,
                 n_group: int = 1, topk_group: int = 1, norm_topk_prob: bool = True, routed_scaling_factor: float = 1.0, tie_word_embeddings: bool = False, ep_size: int = 1):
        super().__init__()
        types = list(layer_types or ["mamba", "moe", "attention", "moe"])
        self.ep_size = ep_size
        self.vocab_size, self.d_model, self.n_layers = vocab_size, d_model, len(types)
        kinds = {"mamba": (NemotronHMambaBlock, dict(d_model=d_model, mamba_num_heads=mamba_num_heads, mamba_head_dim=mamba_head_dim, n_groups=n_groups,
                                                     ssm_state_size=ssm_state_size, conv_kernel=conv_kernel, chunk_size=chunk_size, eps=eps)),
                 "attention": (NemotronHAttentionBlock, dict(d_model=d_model, num_query_heads=num_query_heads, num_kv_heads=num_kv_heads, head_size=head_size, eps=eps)),
                 "moe": (NemotronHMoEBlock, dict(ep_size=ep_size, d_model=d_model, num_experts=num_experts, num_experts_per_tok=num_experts_per_tok, moe_d_ff=moe_d_ff,
                                                 shared_d_ff=shared_d_ff, n_group=n_group, topk_group=topk_group, norm_topk_prob=norm_topk_prob,
                                                 routed_scaling_factor=routed_scaling_factor, eps=eps))}
        unknown = sorted(set(types) - set(kinds))
        if unknown:
            raise ValueError(f"[E021] Nemotron-H layer types {unknown} are not supported (known: {sorted(kinds)})")
        self.embedding = Embedding(vocab_size, d_model, hf_name="backbone.embedding.weight")
        self.blocks = nn.HybridBlockStack(types, {k: v for k, v in kinds.items() if k in types})
        self.final_norm = RMSNorm(d_model, eps=eps, hf_name="backbone.norm_f.weight")
        self.lm_head = LMHead(vocab_size, d_model, tie_to="embedding" if tie_word_embeddings else None)

    def forward(self, token_ids, position_ids, targets):
        x = self.embedding(token_ids)
        residual = F.zeros(("B", "T", self.d_model), name="residual0")
        x, residual = self.blocks(x, residual, position_ids)
        residual, x = self.final_norm(residual, x)
        return self.lm_head(x, targets)

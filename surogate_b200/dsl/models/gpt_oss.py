"""GPT-OSS (``GptOssForCausalLM``): sink attention alternating between sliding-window and full layers, YaRN RoPE, biased MoE.

Parity: surogate/dsl/models/gpt_oss.py.
"""
from __future__ import annotations

from typing import List, Optional

from .. import functional as F
from .. import nn
from ..blocks import STANDARD_MODEL_NAME_REMAP
from ..blocks.gpt_oss import GptOssBlock
from ..modules import Embedding, LMHead, RMSNorm


@nn.hf_config(architecture="GptOssForCausalLM", model_type="gpt_oss", d_model="hidden_size", n_layers="num_hidden_layers",
              num_query_heads="num_attention_heads", num_kv_heads="num_key_value_heads", d_ff="intermediate_size", vocab_size="vocab_size",
              max_seq="max_position_embeddings", head_size="head_dim", eps="rms_norm_eps", rope_theta="rope_theta", num_experts="num_experts",
              num_experts_per_tok="num_experts_per_tok", sliding_window="sliding_window", layer_types="layer_types",
              rope_scaling="rope_parameters", tie_word_embeddings="tie_word_embeddings")
class GptOssModel(nn.Model):
    _name_remap_ = STANDARD_MODEL_NAME_REMAP

    def __init__(self, vocab_size: int = 201088, d_model: int = 2880, n_layers: int = 24, num_query_heads: int = 64, num_kv_heads: int = 8,
                 d_ff: int = 2880, max_seq: int = 131072, head_size: int = 64, eps: float = 1e-5, rope_theta: float = 150000.0, num_experts: int = 32,
                 num_experts_per_tok: int = 4, sliding_window: int = 128, layer_types: Optional[List[str]] = None, rope_scaling=None,
                 tie_word_embeddings: bool = False, ep_size: int = 1):
        super().__init__()
        self.ep_size = ep_size
        self.vocab_size, self.d_model, self.n_layers = vocab_size, d_model, n_layers
        self.num_experts, self.num_experts_per_tok = num_experts, num_experts_per_tok
        types = list(layer_types) if layer_types else ["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(n_layers)]
        scaling = dict(rope_scaling) if isinstance(rope_scaling, dict) and (rope_scaling.get("rope_type") or rope_scaling.get("type", "default")) != "default" else None
        common = dict(d_model=d_model, num_query_heads=num_query_heads, num_kv_heads=num_kv_heads, head_size=head_size, d_ff=d_ff, num_experts=num_experts,
                      num_experts_per_tok=num_experts_per_tok, eps=eps, rope_theta=float(rope_theta), rope_scaling=scaling, max_seq=max_seq, ep_size=ep_size)
        classes = {}
        if "sliding_attention" in types:
            classes["sliding_attention"] = (_named(GptOssBlock, "GptOssSlidingBlock"), dict(common, sliding_window=sliding_window))
        if "full_attention" in types:
            classes["full_attention"] = (_named(GptOssBlock, "GptOssFullBlock"), dict(common, sliding_window=0))
        self.embedding = Embedding(vocab_size, d_model)
        self.blocks = nn.HybridBlockStack(types, classes)
        self.final_norm = RMSNorm(d_model, eps=eps, hf_name="model.norm.weight")
        self.lm_head = LMHead(vocab_size, d_model, tie_to="embedding" if tie_word_embeddings else None)

    def forward(self, token_ids, position_ids, targets):
        x = self.embedding(token_ids)
        residual = F.zeros(("B", "T", self.d_model), name="residual0")
        x, residual = self.blocks(x, residual, position_ids)
        residual, x = self.final_norm(residual, x)
        return self.lm_head(x, targets)


def _named(cls, name):
    return type(name, (cls,), {})

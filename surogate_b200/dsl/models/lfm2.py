"""LFM2 (``Lfm2ForCausalLM``): short-convolution and attention layers interleaved per ``layer_types``.

Parity: surogate/dsl/models/lfm2.py.
"""
from __future__ import annotations

from typing import List, Optional

from .. import functional as F
from .. import nn
from ..blocks import STANDARD_MODEL_NAME_REMAP
from ..blocks.lfm2 import Lfm2AttentionBlock, Lfm2ConvBlock
from ..modules import Embedding, LMHead, RMSNorm


@nn.hf_config(architecture="Lfm2ForCausalLM", model_type="lfm2", d_model="hidden_size", n_layers="num_hidden_layers", num_query_heads="num_attention_heads",
              num_kv_heads="num_key_value_heads", d_ff="intermediate_size", vocab_size="vocab_size", max_seq="max_position_embeddings", eps="norm_eps",
              rope_theta="rope_theta", layer_types="layer_types", conv_kernel="conv_L_cache", conv_bias="conv_bias",
              auto_adjust_ff="block_auto_adjust_ff_dim", ff_multiplier="block_ffn_dim_multiplier", ff_multiple_of="block_multiple_of",
              tie_word_embeddings="tie_word_embeddings")
class Lfm2Model(nn.Model):
    _name_remap_ = STANDARD_MODEL_NAME_REMAP

    def __init__(self, vocab_size: int = 65536, d_model: int = 2560, n_layers: int = 32, num_query_heads: int = 32, num_kv_heads: int = 8,
                 d_ff: int = 12288, max_seq: int = 128000, eps: float = 1e-5, rope_theta: float = 1e6, layer_types: Optional[List[str]] = None,
                 conv_kernel: int = 3, conv_bias: bool = False, auto_adjust_ff: bool = True, ff_multiplier: Optional[float] = 1.0,
                 ff_multiple_of: int = 256, tie_word_embeddings: bool = True):
        super().__init__()
        self.vocab_size, self.d_model, self.n_layers = vocab_size, d_model, n_layers
        if auto_adjust_ff:  # the checkpoint's feed-forward width is derived from intermediate_size this way
            d_ff = int(2 * d_ff / 3)
            if ff_multiplier is not None:
                d_ff = int(ff_multiplier * d_ff)
                d_ff = ff_multiple_of * ((d_ff + ff_multiple_of - 1) // ff_multiple_of)
        self.d_ff = d_ff
        types = list(layer_types) if layer_types else ["conv"] * n_layers
        head = d_model // num_query_heads
        classes = {}
        if "full_attention" in types:
            classes["full_attention"] = (Lfm2AttentionBlock, dict(d_model=d_model, num_query_heads=num_query_heads, num_kv_heads=num_kv_heads, head_size=head,
                                                                   d_ff=d_ff, eps=eps, rope_theta=float(rope_theta), max_seq=max_seq))
        if "conv" in types:
            classes["conv"] = (Lfm2ConvBlock, dict(d_model=d_model, d_ff=d_ff, eps=eps, conv_kernel=conv_kernel, conv_bias=conv_bias))
        self.embedding = Embedding(vocab_size, d_model)
        self.blocks = nn.HybridBlockStack(types, classes)
        self.final_norm = RMSNorm(d_model, eps=eps, hf_name="model.embedding_norm.weight")
        self.lm_head = LMHead(vocab_size, d_model, tie_to="embedding" if tie_word_embeddings else None)

    def forward(self, token_ids, position_ids, targets):
        x = self.embedding(token_ids)
        residual = F.zeros(("B", "T", self.d_model), name="residual0")
        x, residual = self.blocks(x, residual, position_ids)
        residual, x = self.final_norm(residual, x)
        return self.lm_head(x, targets)

"""Qwen3-VL text decoder layer: the Qwen3 dense layer with multi-axis rotary positions (temporal / height / width, interleaved
over the frequency index) and "deepstack": the first few layers add an intermediate vision-tower feature to the hidden state at
the image / video token positions.

Parity: surogate/dsl/blocks/qwen3_vl.py.
"""
from __future__ import annotations

from .. import functional as F
from ..modules import AttentionConfig, GenericGQAttention, GenericMLP, RMSNorm
from ..nn import Block
from .common import DENSE_BLOCK_NAME_REMAP

_P = "model.language_model.layers.{L}"


class Qwen3VLBlock(Block):
    _name_remap_ = DENSE_BLOCK_NAME_REMAP

    def __init__(self, d_model: int, num_query_heads: int, num_kv_heads: int, head_size: int, d_ff: int, max_seq: int = 0, eps: float = 1e-6,
                 use_qkv_bias: bool = False, rope_theta: float = 5e6, mrope_section=(24, 20, 20)):
        super().__init__()
        self.attn_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.input_layernorm.weight")
        self.self_attn = GenericGQAttention(d_model, num_query_heads, num_kv_heads, head_size, max_seq, prefix=f"{_P}.self_attn",
                                            config=AttentionConfig(qk_norm=True, qkv_bias=use_qkv_bias, eps=eps, rope_theta=rope_theta,
                                                                   mrope_section=tuple(mrope_section)))
        self.mlp_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.post_attention_layernorm.weight")
        self.mlp = GenericMLP(d_model, d_ff, prefix=f"{_P}.mlp")

    def forward(self, x, residual, position_ids):
        residual, h = self.attn_norm(residual, x)
        h = self.self_attn(h, position_ids)
        residual, h = self.mlp_norm(residual, h)
        h = self.mlp(h)
        # hidden = residual + h is formed by the next norm, so adding to h at the visual positions adds to the hidden state
        h = F.torch_fn("deepstack_add", [h], [("mlp_plus_deepstack", h.shape, "act")], side_inputs=["visual_pos_masks", "deepstack_visual_embeds"], pass_layer=True)
        return h, residual

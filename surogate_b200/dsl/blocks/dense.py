"""Dense decoder blocks: pre-norm attention + gated MLP on a residual stream.

The residual add of each sub-layer is fused into the *next* RMSNorm, so a block
receives (x, residual) and returns (mlp_out, residual_after_attention).

Parity: surogate/dsl/blocks/qwen3.py:13-63, blocks/llama.py.
"""
from __future__ import annotations

from ..modules import AttentionConfig, GenericGQAttention, GenericMLP, MLPConfig, RMSNorm
from ..nn import Block
from .common import DENSE_BLOCK_NAME_REMAP

_P = "model.layers.{L}"


class DenseBlock(Block):
    _name_remap_ = DENSE_BLOCK_NAME_REMAP

    def __init__(self, d_model: int, num_query_heads: int, num_kv_heads: int, head_size: int, d_ff: int, max_seq: int = 0,
                 eps: float = 1e-6, use_qkv_bias: bool = False, use_qk_norm: bool = False, rope_theta: float = 1e6,
                 sliding_window: int = 0, rotary_dim: int | None = None, mlp_tile_rows: int = 0):
        super().__init__()
        self.attn_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.input_layernorm.weight")
        self.self_attn = GenericGQAttention(
            d_model, num_query_heads, num_kv_heads, head_size, max_seq,
            config=AttentionConfig(qk_norm=use_qk_norm, qkv_bias=use_qkv_bias, eps=eps, rope_theta=rope_theta,
                                   sliding_window=sliding_window, rotary_dim=rotary_dim))
        self.mlp_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.post_attention_layernorm.weight")
        self.mlp = GenericMLP(d_model, d_ff, config=MLPConfig(tile_rows=mlp_tile_rows))

    def forward(self, x, residual, position_ids):
        residual, h = self.attn_norm(residual, x)
        h = self.self_attn(h, position_ids)
        residual, h = self.mlp_norm(residual, h)
        h = self.mlp(h)
        return h, residual


class Qwen3Block(DenseBlock):
    """Qwen3: per-head QK RMSNorm, no QKV bias."""

    def __init__(self, **kw):
        kw.setdefault("use_qk_norm", True)
        super().__init__(**kw)


class Qwen2Block(DenseBlock):
    """Qwen2 / Qwen2.5: QKV bias, no QK norm."""

    def __init__(self, **kw):
        kw.setdefault("use_qkv_bias", True)
        super().__init__(**kw)


class LlamaBlock(DenseBlock):
    """Llama / Mistral family: no QK norm, no bias."""

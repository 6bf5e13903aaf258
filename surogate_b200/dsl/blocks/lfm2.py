"""LFM2 hybrid blocks: a gated short causal convolution or grouped-query attention (QK-norm + RoPE) as the sequence operator,
followed by a SwiGLU MLP; RMSNorm before each.

Parity: surogate/dsl/blocks/lfm2.py, surogate/dsl/modules (Lfm2ShortConv).
"""
from __future__ import annotations

from .. import functional as F
from .. import hf
from ..modules import AttentionConfig, GenericGQAttention, GenericMLP, RMSNorm
from ..nn import Block, Module
from .common import DENSE_BLOCK_NAME_REMAP

_P = "model.layers.{L}"


class ShortConv(Module):
    def __init__(self, d_model: int, kernel: int, bias: bool, prefix: str = f"{_P}.conv"):
        super().__init__()
        self.kernel, self.bias, self.d_model = kernel, bias, d_model
        self.declare_param("in_weight", (3 * d_model, d_model), hf=hf.direct(f"{prefix}.in_proj.weight"))
        self.declare_param("conv_weight", (d_model, 1, kernel), hf=hf.direct(f"{prefix}.conv.weight"), decay=False)
        self.declare_param("out_weight", (d_model, d_model), hf=hf.direct(f"{prefix}.out_proj.weight"))
        if bias:
            self.declare_param("in_bias", (3 * d_model,), init="zeros", decay=False, hf=hf.direct(f"{prefix}.in_proj.bias"))
            self.declare_param("conv_bias", (d_model,), init="zeros", decay=False, hf=hf.direct(f"{prefix}.conv.bias"))
            self.declare_param("out_bias", (d_model,), init="zeros", decay=False, hf=hf.direct(f"{prefix}.out_proj.bias"))

    def forward(self, x):
        b = [self.p("in_bias"), self.p("conv_bias"), self.p("out_bias")] if self.bias else [None, None, None]
        return F.torch_fn("short_conv", [x, self.p("in_weight"), self.p("conv_weight"), self.p("out_weight")] + b, [("conv_out", x.shape, "act")],
                          kernel=self.kernel)


class _Lfm2Base(Block):
    _name_remap_ = {**DENSE_BLOCK_NAME_REMAP, "conv.*": ""}

    def __init__(self, d_model, d_ff, eps):
        super().__init__()
        self.attn_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.operator_norm.weight")
        self.mlp_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.ffn_norm.weight")
        self.mlp = GenericMLP(d_model, d_ff, prefix=f"{_P}.feed_forward", names=("w3", "w1", "w2"))

    def operator(self, h, position_ids):  # pragma: no cover - abstract
        raise NotImplementedError

    def forward(self, x, residual, position_ids):
        residual, h = self.attn_norm(residual, x)
        h = self.operator(h, position_ids)
        residual, h = self.mlp_norm(residual, h)
        return self.mlp(h), residual


class Lfm2AttentionBlock(_Lfm2Base):
    def __init__(self, d_model, num_query_heads, num_kv_heads, head_size, d_ff, eps=1e-5, rope_theta=1e6, max_seq=0, **_):
        super().__init__(d_model, d_ff, eps)
        self.self_attn = GenericGQAttention(d_model, num_query_heads, num_kv_heads, head_size, max_seq,
                                            config=AttentionConfig(qk_norm=True, eps=eps, rope_theta=rope_theta),
                                            names={"o": "out_proj", "q_norm": "q_layernorm", "k_norm": "k_layernorm"})

    def operator(self, h, position_ids):
        return self.self_attn(h, position_ids)


class Lfm2ConvBlock(_Lfm2Base):
    def __init__(self, d_model, d_ff, eps=1e-5, conv_kernel=3, conv_bias=False, **_):
        super().__init__(d_model, d_ff, eps)
        self.conv = ShortConv(d_model, conv_kernel, conv_bias)

    def operator(self, h, position_ids):
        return self.conv(h)

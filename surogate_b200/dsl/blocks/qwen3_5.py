"""Qwen3.5 hybrid blocks: Gated DeltaNet ("linear_attention") or output-gated attention ("full_attention") followed by a
SwiGLU MLP; all RMSNorms are zero-centred (the checkpoint stores w - 1).

Parity: surogate/dsl/blocks/qwen3_5.py, surogate/dsl/modules (GatedDeltaNetMixer).
"""
from __future__ import annotations

from .. import functional as F
from .. import hf
from ..modules import GenericMLP, RMSNorm
from ..nn import Block, Module
from .common import DENSE_BLOCK_NAME_REMAP

_P = "model.language_model.layers.{L}"  # the text model sits under language_model in these checkpoints


class GatedAttention(Module):
    def __init__(self, d_model, num_query_heads, num_kv_heads, head_size, eps, rope_theta, rotary_dim, prefix=f"{_P}.self_attn"):
        super().__init__()
        self.attrs = dict(num_q_heads=num_query_heads, num_kv_heads=num_kv_heads, head_dim=head_size, eps=eps, rope_theta=rope_theta, rotary_dim=rotary_dim)
        qd, kd = num_query_heads * head_size, num_kv_heads * head_size
        self.declare_param("q_weight", (2 * qd, d_model), hf=hf.direct(f"{prefix}.q_proj.weight"))
        self.declare_param("k_weight", (kd, d_model), hf=hf.direct(f"{prefix}.k_proj.weight"))
        self.declare_param("v_weight", (kd, d_model), hf=hf.direct(f"{prefix}.v_proj.weight"))
        self.declare_param("out_weight", (d_model, qd), hf=hf.direct(f"{prefix}.o_proj.weight"))
        self.declare_param("q_norm_weight", (head_size,), init="zeros", decay=False, hf=hf.direct(f"{prefix}.q_norm.weight"))
        self.declare_param("k_norm_weight", (head_size,), init="zeros", decay=False, hf=hf.direct(f"{prefix}.k_norm.weight"))

    def forward(self, x, position_ids):
        names = ("q_weight", "k_weight", "v_weight", "out_weight", "q_norm_weight", "k_norm_weight")
        return F.torch_fn("qwen35_gated_attention", [x] + [self.p(n) for n in names] + [position_ids], [("att_out", x.shape, "act")], **self.attrs)


class GatedDeltaNet(Module):
    def __init__(self, d_model, num_k_heads, num_v_heads, head_k_dim, head_v_dim, conv_kernel, eps, prefix=f"{_P}.linear_attn"):
        super().__init__()
        self.attrs = dict(num_k_heads=num_k_heads, num_v_heads=num_v_heads, head_k_dim=head_k_dim, head_v_dim=head_v_dim, conv_kernel=conv_kernel, eps=eps)
        key_dim, value_dim = num_k_heads * head_k_dim, num_v_heads * head_v_dim
        conv_dim = 2 * key_dim + value_dim
        self.declare_param("qkv_weight", (conv_dim, d_model), hf=hf.direct(f"{prefix}.in_proj_qkv.weight"))
        self.declare_param("z_weight", (value_dim, d_model), hf=hf.direct(f"{prefix}.in_proj_z.weight"))
        self.declare_param("b_weight", (num_v_heads, d_model), hf=hf.direct(f"{prefix}.in_proj_b.weight"))
        self.declare_param("a_weight", (num_v_heads, d_model), hf=hf.direct(f"{prefix}.in_proj_a.weight"))
        self.declare_param("conv_weight", (conv_dim, 1, conv_kernel), decay=False, hf=hf.direct(f"{prefix}.conv1d.weight"))
        self.declare_param("dt_bias", (num_v_heads,), init="ones", decay=False, hf=hf.direct(f"{prefix}.dt_bias"))
        self.declare_param("A_log", (num_v_heads,), init="ones", decay=False, hf=hf.direct(f"{prefix}.A_log"))
        self.declare_param("gdn_norm_weight", (head_v_dim,), init="ones", decay=False, hf=hf.direct(f"{prefix}.norm.weight"))
        self.declare_param("out_weight", (d_model, value_dim), hf=hf.direct(f"{prefix}.out_proj.weight"))

    def forward(self, x):
        names = ("qkv_weight", "z_weight", "b_weight", "a_weight", "conv_weight", "dt_bias", "A_log", "gdn_norm_weight", "out_weight")
        return F.torch_fn("qwen35_gated_delta_net", [x] + [self.p(n) for n in names], [("gdn_out", x.shape, "act")], **self.attrs)


class _Qwen35Base(Block):
    _name_remap_ = {**DENSE_BLOCK_NAME_REMAP, "linear_attn.*": ""}

    def __init__(self, d_model, d_ff, eps):
        super().__init__()
        self.attn_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.input_layernorm.weight", zero_centered=True)
        self.mlp_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.post_attention_layernorm.weight", zero_centered=True)
        self.mlp = GenericMLP(d_model, d_ff, prefix=f"{_P}.mlp")

    def forward(self, x, residual, position_ids):
        residual, h = self.attn_norm(residual, x)
        h = self.operator(h, position_ids)
        residual, h = self.mlp_norm(residual, h)
        return self.mlp(h), residual


class Qwen35AttentionBlock(_Qwen35Base):
    def __init__(self, d_model, d_ff, num_query_heads, num_kv_heads, head_size, eps, rope_theta, rotary_dim, **_):
        super().__init__(d_model, d_ff, eps)
        self.self_attn = GatedAttention(d_model, num_query_heads, num_kv_heads, head_size, eps, rope_theta, rotary_dim)

    def operator(self, h, position_ids):
        return self.self_attn(h, position_ids)


class Qwen35LinearBlock(_Qwen35Base):
    def __init__(self, d_model, d_ff, num_k_heads, num_v_heads, head_k_dim, head_v_dim, conv_kernel, eps, **_):
        super().__init__(d_model, d_ff, eps)
        self.linear_attn = GatedDeltaNet(d_model, num_k_heads, num_v_heads, head_k_dim, head_v_dim, conv_kernel, eps)

    def operator(self, h, position_ids):
        return self.linear_attn(h)


class _Qwen35MoEBase(Block):
    """Qwen3.5-MoE layer: the same two token mixers, followed by routed experts plus a sigmoid-gated shared expert.
    Returns (y, residual, aux_loss).  Parity: surogate/dsl/blocks/qwen3_5_moe.py."""
    _name_remap_ = {**DENSE_BLOCK_NAME_REMAP, "linear_attn.*": ""}

    def __init__(self, d_model, moe_d_ff, shared_d_ff, num_experts, num_experts_per_tok, norm_topk_prob, ep_size, aux_loss_coef, eps):
        super().__init__()
        from ..modules import MoEExpertsGated, MoESharedExpert

        self.attn_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.input_layernorm.weight", zero_centered=True)
        self.mlp_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.post_attention_layernorm.weight", zero_centered=True)
        self.mlp = MoEExpertsGated(d_model, moe_d_ff, num_experts, num_experts_per_tok, norm_topk_prob, ep_size, aux_loss_coef,
                                   prefix=f"{_P}.mlp")  # saved checkpoints list every expert separately
        self.has_shared = shared_d_ff > 0
        if self.has_shared:
            self.shared_expert = MoESharedExpert(d_model, shared_d_ff, prefix=f"{_P}.mlp.shared_expert", gate_name=f"{_P}.mlp.shared_expert_gate.weight")

    def forward(self, x, residual, position_ids):
        residual, h = self.attn_norm(residual, x)
        h = self.operator(h, position_ids)
        residual, h = self.mlp_norm(residual, h)
        y, aux = self.mlp(h)
        if self.has_shared:
            y = F.add(y, self.shared_expert(h), name="moe_plus_shared")
        return y, residual, aux


class Qwen35MoEAttentionBlock(_Qwen35MoEBase):
    def __init__(self, num_query_heads, num_kv_heads, head_size, rope_theta, rotary_dim, **kw):
        super().__init__(**kw)
        self.self_attn = GatedAttention(kw["d_model"], num_query_heads, num_kv_heads, head_size, kw["eps"], rope_theta, rotary_dim)

    def operator(self, h, position_ids):
        return self.self_attn(h, position_ids)


class Qwen35MoELinearBlock(_Qwen35MoEBase):
    def __init__(self, num_k_heads, num_v_heads, head_k_dim, head_v_dim, conv_kernel, **kw):
        super().__init__(**kw)
        self.linear_attn = GatedDeltaNet(kw["d_model"], num_k_heads, num_v_heads, head_k_dim, head_v_dim, conv_kernel, kw["eps"])

    def operator(self, h, position_ids):
        return self.linear_attn(h)

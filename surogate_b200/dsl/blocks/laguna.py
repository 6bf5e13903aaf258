"""Laguna decoder layers: QK-normed GQA attention with a softplus output gate (full or sliding-window, each with its own
rotary setup and query-head count), followed by a dense SwiGLU MLP or by routed experts (sigmoid router with a selection-only
correction bias, renormalised and scaled top-k weights) plus an ungated shared expert.

Parity: surogate/dsl/blocks/laguna.py (LagunaDenseBlock, LagunaSparseBlock), surogate/dsl/modules/attention.py (LagunaAttention),
surogate/dsl/modules/moe.py (LagunaMoEExperts).
"""
from __future__ import annotations

from .. import functional as F
from .. import hf
from ..modules import AttentionConfig, GenericGQAttention, GenericMLP, MoESharedExpert, RMSNorm
from ..nn import Block, Module
from .common import DENSE_BLOCK_NAME_REMAP

_P = "model.layers.{L}"


class LagunaExperts(Module):
    def __init__(self, d_model: int, d_ff: int, num_experts: int, top_k: int, routed_scaling_factor: float = 1.0, ep_size: int = 1, prefix: str = f"{_P}.mlp"):
        super().__init__()
        self.E, self.K, self.scale, self.ep_size = num_experts, top_k, routed_scaling_factor, ep_size
        m = prefix
        self.declare_param("router_weight", (num_experts, d_model), hf=hf.direct(f"{m}.gate.weight"))
        # selection-only bias (a buffer in the checkpoint, stored beside the experts); it never receives a gradient
        self.declare_param("e_score_correction_bias", (num_experts,), init="zeros", decay=False, hf=hf.direct(f"{m}.experts.e_score_correction_bias"))
        self.declare_param("experts_gate_up", (num_experts, 2 * d_ff, d_model), quantizable=True,
                           hf=hf.stack_experts([f"{m}.experts.{{E}}.up_proj.weight", f"{m}.experts.{{E}}.gate_proj.weight"], num_experts, sizes=[d_ff, d_ff]),
                           lora_targets=[("up_proj", 0, d_ff), ("gate_proj", d_ff, d_ff)])
        self.declare_param("experts_down", (num_experts, d_model, d_ff), quantizable=True,
                           hf=hf.stack_experts([f"{m}.experts.{{E}}.down_proj.weight"], num_experts), lora_targets=[("down_proj", 0, d_model)])

    def forward(self, x):
        lead = x.shape[:-1]
        tw, ti = F.torch_fn("sigmoid_bias_router", [x, self.p("router_weight"), self.p("e_score_correction_bias")],
                            [("topk_weights", lead + (self.K,), "fp32"), ("topk_index", lead + (self.K,), "int32")], top_k=self.K, scaling_factor=self.scale)
        xp, plan = F.moe_permute(x, ti, num_experts=self.E, top_k=self.K)
        if self.ep_size > 1:
            xp, plan = F.ep_dispatch(xp, plan)
        h = F.moe_grouped_gemm(xp, self.p("experts_gate_up"), plan, name="moe_gate_up", role="experts_gate_up")
        h = F.swiglu(h, name="moe_swiglu")
        h = F.moe_grouped_gemm(h, self.p("experts_down"), plan, name="moe_down", role="experts_down")
        if self.ep_size > 1:
            h = F.ep_combine(h, plan)
        return F.moe_unpermute(h, tw, plan, x.shape)


class _LagunaBase(Block):
    _name_remap_ = DENSE_BLOCK_NAME_REMAP

    def __init__(self, d_model, num_query_heads, num_kv_heads, head_size, max_seq, sliding_window, rope_theta, rotary_dim, rope_scaling, gate_per_head, eps):
        super().__init__()
        self.attn_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.input_layernorm.weight")
        self.self_attn = GenericGQAttention(
            d_model, num_query_heads, num_kv_heads, head_size, max_seq,
            config=AttentionConfig(qk_norm=True, eps=eps, rope_theta=rope_theta, rotary_dim=rotary_dim, sliding_window=int(sliding_window or 0),
                                   rope_scaling=rope_scaling, max_pos=max_seq if rope_scaling else None,
                                   output_gate="softplus_head" if gate_per_head else "softplus_element"))
        self.mlp_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.post_attention_layernorm.weight")

    def forward(self, x, residual, position_ids):
        residual, h = self.attn_norm(residual, x)
        h = self.self_attn(h, position_ids)
        residual, h = self.mlp_norm(residual, h)
        return self.feed_forward(h), residual


class LagunaDenseBlock(_LagunaBase):
    def __init__(self, d_ff, **kw):
        super().__init__(**kw)
        self.mlp = GenericMLP(kw["d_model"], d_ff)

    def feed_forward(self, h):
        return self.mlp(h)


class LagunaSparseBlock(_LagunaBase):
    def __init__(self, moe_d_ff, num_experts, num_experts_per_tok, shared_d_ff, routed_scaling_factor=1.0, ep_size=1, **kw):
        super().__init__(**kw)
        self.mlp = LagunaExperts(kw["d_model"], moe_d_ff, num_experts, num_experts_per_tok, routed_scaling_factor, ep_size)
        self.shared_expert = MoESharedExpert(kw["d_model"], shared_d_ff, prefix=f"{_P}.mlp.shared_expert") if shared_d_ff else None

    def feed_forward(self, h):
        y = self.mlp(h)
        if self.shared_expert is not None:
            y = F.add(y, self.shared_expert(h), name="moe_plus_shared")
        return y

"""GPT-OSS decoder block: biased GQA attention with learned sink logits and alternating sliding-window / full layers,
then a mixture of experts whose router is a biased linear layer (top-k, softmax over the selected logits) and whose
experts use interleaved (gate, up) columns, clamping and the ``(up + 1) * gate * sigmoid(alpha * gate)`` activation.

The attention core and the expert mixture run through the generic PyTorch-function op; the projections are ordinary
``matmul`` ops, so recipes and LoRA apply to them.

Parity: surogate/dsl/blocks/gpt_oss.py, surogate/dsl/models/gpt_oss.py.
"""
from __future__ import annotations

from .. import functional as F
from .. import hf
from ..modules import RMSNorm
from ..nn import Block, Module
from .common import DENSE_BLOCK_NAME_REMAP

_P = "model.layers.{L}"


class SinkAttention(Module):
    def __init__(self, d_model, num_query_heads, num_kv_heads, head_size, window, rope_theta, rope_scaling, max_seq, prefix=f"{_P}.self_attn"):
        super().__init__()
        self.Hq, self.Hkv, self.D, self.window = num_query_heads, num_kv_heads, head_size, window
        self.rope_theta, self.rope_scaling, self.max_seq = rope_theta, rope_scaling, max_seq
        qd, kd, a = num_query_heads * head_size, num_kv_heads * head_size, prefix
        self.declare_param("qkv_weight", (qd + 2 * kd, d_model), quantizable=True,
                           hf=hf.fuse([f"{a}.q_proj.weight", f"{a}.k_proj.weight", f"{a}.v_proj.weight"], sizes=[qd, kd, kd]),
                           lora_targets=[("q_proj", 0, qd), ("k_proj", qd, kd), ("v_proj", qd + kd, kd)])
        self.declare_param("qkv_bias", (qd + 2 * kd,), init="zeros", decay=False,
                           hf=hf.fuse([f"{a}.q_proj.bias", f"{a}.k_proj.bias", f"{a}.v_proj.bias"], sizes=[qd, kd, kd]))
        self.declare_param("out_weight", (d_model, qd), quantizable=True, hf=hf.direct(f"{a}.o_proj.weight"), lora_targets=[("o_proj", 0, d_model)])
        self.declare_param("out_bias", (d_model,), init="zeros", decay=False, hf=hf.direct(f"{a}.o_proj.bias"))
        self.declare_param("sinks", (num_query_heads,), init="normal", decay=False, hf=hf.direct(f"{a}.sinks"))

    def forward(self, x, position_ids):
        qkv = F.matmul(x, self.p("qkv_weight"), self.p("qkv_bias"), name="qkv", role="qkv")
        qkv, _, _ = F.qkv_qk_norm_rope(qkv, None, None, position_ids, num_q_heads=self.Hq, num_kv_heads=self.Hkv, head_dim=self.D, eps=0.0,
                                       rope_theta=self.rope_theta, rope_scaling=self.rope_scaling, max_pos=self.max_seq)
        att = F.torch_fn("attention_general", [qkv, self.p("sinks")], [("att", qkv.shape[:-1] + (self.Hq * self.D,), "act")],
                         num_q_heads=self.Hq, num_kv_heads=self.Hkv, head_dim=self.D, window=self.window)
        return F.matmul(att, self.p("out_weight"), self.p("out_bias"), name="att_out", role="out")


class BiasedClampMoE(Module):
    """Router with bias and softmax over the chosen logits; experts with biases, interleaved gate / up columns and the clamped
    activation.  The checkpoint stores expert weights input-major ([E, C, 2M], [E, M, C]); they are kept output-major here
    (transposed on load / export) so that the experts run on the grouped GEMM path, expert-parallel when ``ep_size`` > 1."""

    def __init__(self, d_model, d_ff, num_experts, top_k, alpha=1.702, limit=7.0, prefix=f"{_P}.mlp", ep_size=1):
        super().__init__()
        self.E, self.top_k, self.alpha, self.limit, self.ep_size = num_experts, top_k, alpha, limit, ep_size
        self.declare_param("router_weight", (num_experts, d_model), hf=hf.direct(f"{prefix}.router.weight"))
        self.declare_param("router_bias", (num_experts,), init="zeros", decay=False, hf=hf.direct(f"{prefix}.router.bias"))
        self.declare_param("experts_gate_up", (num_experts, 2 * d_ff, d_model), quantizable=True, hf=hf.transform(f"{prefix}.experts.gate_up_proj", fn="transpose"))
        self.declare_param("experts_gate_up_bias", (num_experts, 2 * d_ff), init="zeros", decay=False, hf=hf.direct(f"{prefix}.experts.gate_up_proj_bias"))
        self.declare_param("experts_down", (num_experts, d_model, d_ff), quantizable=True, hf=hf.transform(f"{prefix}.experts.down_proj", fn="transpose"))
        self.declare_param("experts_down_bias", (num_experts, d_model), init="zeros", decay=False, hf=hf.direct(f"{prefix}.experts.down_proj_bias"))

    def forward(self, x):
        lead = x.shape[:-1]
        tw, ti = F.torch_fn("topk_softmax_router", [x, self.p("router_weight"), self.p("router_bias")],
                            [("topk_weights", lead + (self.top_k,), "fp32"), ("topk_index", lead + (self.top_k,), "int32")], top_k=self.top_k)
        xp, plan = F.moe_permute(x, ti, num_experts=self.E, top_k=self.top_k)
        if self.ep_size > 1:
            xp, plan = F.ep_dispatch(xp, plan)
        h = F.moe_grouped_gemm(xp, self.p("experts_gate_up"), plan, name="moe_gate_up", role="experts_gate_up")
        h = F.moe_expert_bias_add(h, self.p("experts_gate_up_bias"), plan, name="moe_gate_up_biased")
        h = F.torch_fn("clamped_glu_interleaved", [h], [("moe_act", h.shape[:-1] + (h.shape[-1] // 2,), "act")], alpha=self.alpha, limit=self.limit)
        h = F.moe_grouped_gemm(h, self.p("experts_down"), plan, name="moe_down", role="experts_down")
        h = F.moe_expert_bias_add(h, self.p("experts_down_bias"), plan, name="moe_down_biased")
        if self.ep_size > 1:
            h = F.ep_combine(h, plan)
        return F.moe_unpermute(h, tw, plan, x.shape)


class GptOssBlock(Block):
    _name_remap_ = {**DENSE_BLOCK_NAME_REMAP, "mlp.*": ""}

    def __init__(self, d_model, num_query_heads, num_kv_heads, head_size, d_ff, num_experts, num_experts_per_tok, eps=1e-5, rope_theta=150000.0,
                 rope_scaling=None, sliding_window=0, max_seq=131072, ep_size=1):
        super().__init__()
        self.attn_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.input_layernorm.weight")
        self.self_attn = SinkAttention(d_model, num_query_heads, num_kv_heads, head_size, sliding_window, rope_theta, rope_scaling, max_seq)
        self.mlp_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.post_attention_layernorm.weight")
        self.mlp = BiasedClampMoE(d_model, d_ff, num_experts, num_experts_per_tok, ep_size=ep_size)

    def forward(self, x, residual, position_ids):
        residual, h = self.attn_norm(residual, x)
        h = self.self_attn(h, position_ids)
        residual, h = self.mlp_norm(residual, h)
        return self.mlp(h), residual

"""Gemma4 decoder layers.

Every sub-layer is wrapped in two RMSNorms (before and after), attention has no softmax scaling (q and k are RMS-normalised
per head, v is normalised without a scale), sliding and full layers differ in head size, rotary setup and (with
``attention_k_eq_v``) in full layers reusing the key projection as values; the feed-forward is GeGLU, optionally with routed
experts running in parallel on the same input; a per-layer buffer scales the layer's output.

Parity: surogate/dsl/blocks/gemma4.py (Gemma4SlidingBlock, Gemma4FullBlock, Gemma4*MoEBlock).
"""
from __future__ import annotations

from .. import functional as F
from .. import hf
from ..modules import GenericMLP, MLPConfig, RMSNorm
from ..nn import Block, Module
from .common import DENSE_BLOCK_NAME_REMAP

_P = "model.layers.{L}"


class Gemma4Attention(Module):
    """``kv_role``: "" (own keys / values), "producer" (own, and published under ``kv_key`` for later layers) or "shared"
    (queries only; keys / values come from the producer of the same attention kind, the layer's own k / v weights stay
    untouched in the checkpoint)."""

    def __init__(self, d_model, num_query_heads, num_kv_heads, head_size, window, rope_theta, rope_scaling, k_eq_v, eps, prefix=f"{_P}.self_attn",
                 kv_role: str = "", kv_key: str = ""):
        super().__init__()
        self.kv_role, self.kv_key = kv_role, kv_key
        self.Hq, self.Hkv, self.D, self.window, self.k_eq_v = num_query_heads, num_kv_heads, head_size, int(window or 0), bool(k_eq_v)
        self.fn_attrs = dict(num_q_heads=num_query_heads, num_kv_heads=num_kv_heads, head_dim=head_size, eps=eps, rope_theta=float(rope_theta),
                             rope_scaling=dict(rope_scaling) if rope_scaling else None, k_eq_v=self.k_eq_v)
        qd, kd = num_query_heads * head_size, num_kv_heads * head_size
        a = prefix
        if self.k_eq_v:  # no v_proj in the checkpoint: values are the (separately normalised) keys
            self.declare_param("qkv_weight", (qd + kd, d_model), quantizable=True, hf=hf.fuse([f"{a}.q_proj.weight", f"{a}.k_proj.weight"], sizes=[qd, kd]),
                               lora_targets=[("q_proj", 0, qd), ("k_proj", qd, kd)])
        else:
            self.declare_param("qkv_weight", (qd + 2 * kd, d_model), quantizable=True,
                               hf=hf.fuse([f"{a}.q_proj.weight", f"{a}.k_proj.weight", f"{a}.v_proj.weight"], sizes=[qd, kd, kd]),
                               lora_targets=[("q_proj", 0, qd), ("k_proj", qd, kd), ("v_proj", qd + kd, kd)])
        self.declare_param("out_weight", (d_model, qd), quantizable=True, hf=hf.direct(f"{a}.o_proj.weight"), lora_targets=[("o_proj", 0, d_model)])
        self.declare_param("q_norm_weight", (head_size,), init="ones", decay=False, hf=hf.direct(f"{a}.q_norm.weight"))
        self.declare_param("k_norm_weight", (head_size,), init="ones", decay=False, hf=hf.direct(f"{a}.k_norm.weight"))

    def forward(self, x, position_ids):
        packed = x.shape[:-1] + ((self.Hq + 2 * self.Hkv) * self.D,)
        if self.kv_role == "shared":
            qd = self.Hq * self.D
            x = F.torch_fn("keep_params", [x, self.p("k_norm_weight")], [("x_keep", x.shape, "act")])
            qkv_all = F.matmul(x, self.p("qkv_weight"), name="qkv", role="qkv")  # the k / v columns are computed and dropped: one fused weight per layer kind
            q = F.torch_fn("slice_last", [qkv_all], [("q_only", x.shape[:-1] + (qd,), "act")], start=0, size=qd)
            attrs = {k: v for k, v in self.fn_attrs.items() if k != "k_eq_v"}
            qkv = F.torch_fn("gemma4_q_norm_rope_shared", [q, self.p("q_norm_weight"), position_ids], [("qkv_rope", packed, "act")], shared_in=[self.kv_key], **attrs)
        else:
            qkv = F.matmul(x, self.p("qkv_weight"), name="qkv", role="qkv")
            extra = {"shared_out": [[self.kv_key, 0]]} if self.kv_role == "producer" else {}
            qkv = F.torch_fn("gemma4_qkv_norm_rope", [qkv, self.p("q_norm_weight"), self.p("k_norm_weight"), position_ids], [("qkv_rope", packed, "act")],
                             **self.fn_attrs, **extra)
        att, _ = F.flash_attention(qkv, num_q_heads=self.Hq, num_kv_heads=self.Hkv, head_dim=self.D, causal=True, window=self.window, softmax_scale=1.0)
        return F.matmul(att, self.p("out_weight"), name="att_out", role="out")


class Gemma4Experts(Module):
    """Routed GeGLU experts; the checkpoint stores them as two 3-D tensors with the gate rows first."""

    def __init__(self, d_model, d_ff, num_experts, top_k, eps, ep_size=1, prefix=_P):
        super().__init__()
        self.E, self.K, self.eps, self.ep_size = num_experts, top_k, eps, ep_size
        self.declare_param("router_weight", (num_experts, d_model), hf=hf.direct(f"{prefix}.router.proj.weight"))
        self.declare_param("router_scale", (d_model,), init="ones", decay=False, hf=hf.direct(f"{prefix}.router.scale"))
        self.declare_param("router_per_expert_scale", (num_experts,), init="ones", decay=False, hf=hf.direct(f"{prefix}.router.per_expert_scale"))
        self.declare_param("experts_gate_up", (num_experts, 2 * d_ff, d_model), quantizable=True,
                           hf=hf.transform(f"{prefix}.experts.gate_up_proj", fn="swap_row_halves"), lora_targets=[("up_proj", 0, d_ff), ("gate_proj", d_ff, d_ff)])
        self.declare_param("experts_down", (num_experts, d_model, d_ff), quantizable=True, hf=hf.direct(f"{prefix}.experts.down_proj"),
                           lora_targets=[("down_proj", 0, d_model)])

    def forward(self, router_in, x):
        lead = x.shape[:-1]
        tw, ti = F.torch_fn("gemma4_router", [router_in, self.p("router_weight"), self.p("router_scale"), self.p("router_per_expert_scale")],
                            [("topk_weights", lead + (self.K,), "fp32"), ("topk_index", lead + (self.K,), "int32")], top_k=self.K, eps=self.eps)
        xp, plan = F.moe_permute(x, ti, num_experts=self.E, top_k=self.K)
        if self.ep_size > 1:
            xp, plan = F.ep_dispatch(xp, plan)
        h = F.moe_grouped_gemm(xp, self.p("experts_gate_up"), plan, name="moe_gate_up", role="experts_gate_up")
        h = F.torch_fn("geglu", [h], [("moe_geglu", h.shape[:-1] + (h.shape[-1] // 2,), "act")], approximate="tanh")
        h = F.moe_grouped_gemm(h, self.p("experts_down"), plan, name="moe_down", role="experts_down")
        if self.ep_size > 1:
            h = F.ep_combine(h, plan)
        return F.moe_unpermute(h, tw, plan, x.shape)


class Gemma4Block(Block):
    """One decoder layer; ``moe=True`` adds the parallel expert branch."""
    _name_remap_ = DENSE_BLOCK_NAME_REMAP

    def __init__(self, d_model, num_query_heads, num_kv_heads, head_size, d_ff, window=0, rope_theta=10000.0, rope_scaling=None, k_eq_v=False, eps=1e-6,
                 moe=False, moe_d_ff=0, num_experts=0, top_k=0, ep_size=1, kv_role="", kv_key="", d_pli=0):
        super().__init__()
        self.eps, self.d_pli = eps, int(d_pli)
        self.attn_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.input_layernorm.weight")
        self.self_attn = Gemma4Attention(d_model, num_query_heads, num_kv_heads, head_size, window, rope_theta, rope_scaling, k_eq_v, eps,
                                         kv_role=kv_role, kv_key=kv_key)
        if self.d_pli:
            self.declare_param("pli_gate_weight", (self.d_pli, d_model), hf=hf.direct(f"{_P}.per_layer_input_gate.weight"))
            self.declare_param("pli_proj_weight", (d_model, self.d_pli), hf=hf.direct(f"{_P}.per_layer_projection.weight"))
            self.declare_param("pli_norm_weight", (d_model,), init="ones", decay=False, hf=hf.direct(f"{_P}.post_per_layer_input_norm.weight"))
        self.post_attn_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.post_attention_layernorm.weight", out_name="post_attn_ln")
        self.mlp_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.pre_feedforward_layernorm.weight")
        self.mlp = GenericMLP(d_model, d_ff, config=MLPConfig(activation="geglu"))
        self.post_mlp_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.post_feedforward_layernorm.weight", out_name="post_mlp_ln")
        self.moe = bool(moe)
        if self.moe:
            self.post_mlp_norm_1 = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.post_feedforward_layernorm_1.weight", out_name="post_mlp_ln_1")
            self.pre_moe_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.pre_feedforward_layernorm_2.weight", out_name="pre_moe_ln")
            self.post_moe_norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.post_feedforward_layernorm_2.weight", out_name="post_moe_ln")
            self.experts = Gemma4Experts(d_model, moe_d_ff, num_experts, top_k, eps, ep_size)
        self.declare_param("layer_scalar", (1,), init="ones", decay=False, hf=hf.direct(f"{_P}.layer_scalar"))

    def forward(self, x, residual, position_ids):
        stream, h = self.attn_norm(residual, x)               # stream = residual + x
        a = self.post_attn_norm(self.self_attn(h, position_ids))
        stream, h = self.mlp_norm(stream, a)                  # stream += attention branch
        m = self.mlp(h)
        if self.moe:
            m1 = self.post_mlp_norm_1(m)
            m2 = self.post_moe_norm(self.experts(stream, self.pre_moe_norm(stream)))  # router and experts read the un-normalised stream
            m = F.add(m1, m2, name="mlp_plus_moe")
        m = self.post_mlp_norm(m)
        if self.d_pli:  # the per-layer input acts on the hidden state after the feed-forward residual add
            stream = F.add(stream, m, name="hidden_after_mlp")
            m = F.torch_fn("gemma4_pli_apply", [stream, self.p("pli_gate_weight"), self.p("pli_proj_weight"), self.p("pli_norm_weight")],
                           [("pli_out", stream.shape, "act")], pass_layer=True, shared_in=["pli"], eps=self.eps)
        s = self.p("layer_scalar")
        out = F.torch_fn("scale_by_buffer", [m, s], [("mlp_scaled", m.shape, "act")])
        stream = F.torch_fn("scale_by_buffer", [stream, s], [("stream_scaled", stream.shape, "act")])
        return out, stream

"""Grouped-query attention with fused QKV, optional per-head QK RMSNorm and rotary embedding.

Parity: surogate/dsl/modules/attention.py:51-320 (GenericGQAttention).
"""
from __future__ import annotations

from dataclasses import dataclass

from .. import functional as F
from .. import hf
from ..nn import Module


@dataclass
class AttentionConfig:
    qk_norm: bool = True
    qkv_bias: bool = False
    eps: float = 1e-6
    rope_theta: float = 1e6
    rotary_dim: int | None = None
    sliding_window: int = 0
    causal: bool = True
    mrope_section: tuple | None = None  # (t, h, w) frequency split for multi-axis rotary positions (vision-language models)
    rope_scaling: dict | None = None    # {"rope_type": "yarn" | "linear" | "llama3" | "dynamic", ...}
    max_pos: int | None = None
    output_gate: str = ""               # "" | "softplus_head" | "softplus_element": y *= softplus(x @ g_proj^T) before o_proj


class GenericGQAttention(Module):
    def __init__(self, d_model: int, num_query_heads: int, num_kv_heads: int, head_size: int, max_seq: int = 0,
                 config: AttentionConfig | None = None, prefix: str = "model.layers.{L}.self_attn", names: dict | None = None):
        super().__init__()
        self.cfg = config or AttentionConfig()
        self.Hq, self.Hkv, self.D = num_query_heads, num_kv_heads, head_size
        qd, kd = num_query_heads * head_size, num_kv_heads * head_size
        a = prefix
        n = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "q_norm": "q_norm", "k_norm": "k_norm", **(names or {})}  # checkpoint leaf names
        self.declare_param(
            "qkv_weight", (qd + 2 * kd, d_model), quantizable=True,
            hf=hf.fuse([f"{a}.{n['q']}.weight", f"{a}.{n['k']}.weight", f"{a}.{n['v']}.weight"], sizes=[qd, kd, kd]),
            lora_targets=[("q_proj", 0, qd), ("k_proj", qd, kd), ("v_proj", qd + kd, kd)])
        if self.cfg.qkv_bias:
            self.declare_param("qkv_bias", (qd + 2 * kd,), init="zeros", decay=False,
                               hf=hf.fuse([f"{a}.{n['q']}.bias", f"{a}.{n['k']}.bias", f"{a}.{n['v']}.bias"], sizes=[qd, kd, kd]))
        self.declare_param("out_weight", (d_model, qd), quantizable=True, hf=hf.direct(f"{a}.{n['o']}.weight"),
                           lora_targets=[("o_proj", 0, d_model)])
        if self.cfg.output_gate:
            gate_dim = num_query_heads if self.cfg.output_gate == "softplus_head" else qd
            self.declare_param("g_weight", (gate_dim, d_model), hf=hf.direct(f"{a}.g_proj.weight"))
        if self.cfg.qk_norm:
            self.declare_param("q_norm_weight", (head_size,), init="ones", decay=False, hf=hf.direct(f"{a}.{n['q_norm']}.weight"))
            self.declare_param("k_norm_weight", (head_size,), init="ones", decay=False, hf=hf.direct(f"{a}.{n['k_norm']}.weight"))

    def forward(self, x, position_ids):
        c = self.cfg
        qkv = F.matmul(x, self.p("qkv_weight"), self.p("qkv_bias") if c.qkv_bias else None, name="qkv", role="qkv")
        qn = self.p("q_norm_weight") if c.qk_norm else None
        kn = self.p("k_norm_weight") if c.qk_norm else None
        qkv_rope, _, _ = F.qkv_qk_norm_rope(qkv, qn, kn, position_ids, num_q_heads=self.Hq, num_kv_heads=self.Hkv,
                                            head_dim=self.D, eps=c.eps, rope_theta=c.rope_theta, rotary_dim=c.rotary_dim,
                                            mrope_section=c.mrope_section, rope_scaling=c.rope_scaling, max_pos=c.max_pos)
        att, _ = F.flash_attention(qkv_rope, num_q_heads=self.Hq, num_kv_heads=self.Hkv, head_dim=self.D,
                                   causal=c.causal, window=c.sliding_window)
        if c.output_gate:
            gate = F.matmul(x, self.p("g_weight"), name="att_gate", role="att_gate")
            att = F.torch_fn("softplus_gate_mul", [att, gate], [("att_gated", att.shape, "act")], head_dim=self.D)
        return F.matmul(att, self.p("out_weight"), name="att_out", role="out")

"""Nemotron-H blocks: every layer is ONE mixer behind a pre-norm and a residual add — a Mamba-2 state-space mixer, grouped-query
attention without positional encoding, or a mixture of ReLU^2 experts with a sigmoid router and a shared expert.

Parity: surogate/dsl/blocks/nemotron_h.py, surogate/dsl/modules (Mamba2Mixer).
"""
from __future__ import annotations

from .. import functional as F
from .. import hf
from ..modules import RMSNorm
from ..nn import Block
from .common import DENSE_BLOCK_NAME_REMAP

_P = "backbone.layers.{L}"
_M = f"{_P}.mixer"


class _MixerBlock(Block):
    _name_remap_ = {"norm.weight": "ln1_weight", "norm.ln": "ln1", "norm.ln_rstd": "ln1_rstd", "norm.res": "res_in"}

    def __init__(self, d_model, eps):
        super().__init__()
        self.norm = RMSNorm(d_model, eps=eps, hf_name=f"{_P}.norm.weight")

    def mixer(self, h, position_ids):  # pragma: no cover - abstract
        raise NotImplementedError

    def forward(self, x, residual, position_ids):
        residual, h = self.norm(residual, x)
        return self.mixer(h, position_ids), residual


class NemotronHMambaBlock(_MixerBlock):
    def __init__(self, d_model, mamba_num_heads, mamba_head_dim, n_groups, ssm_state_size, conv_kernel=4, chunk_size=128, eps=1e-5, **_):
        super().__init__(d_model, eps)
        H, P, G, N = mamba_num_heads, mamba_head_dim, n_groups, ssm_state_size
        inner, conv_dim = H * P, H * P + 2 * G * N
        self.attrs = dict(num_heads=H, head_dim=P, n_groups=G, state_size=N, conv_kernel=conv_kernel, chunk=chunk_size, eps=eps)
        self.declare_param("in_weight", (inner + conv_dim + H, d_model), hf=hf.direct(f"{_M}.in_proj.weight"), quantizable=True)
        self.declare_param("conv_weight", (conv_dim, 1, conv_kernel), hf=hf.direct(f"{_M}.conv1d.weight"), decay=False)
        self.declare_param("conv_bias", (conv_dim,), init="zeros", decay=False, hf=hf.direct(f"{_M}.conv1d.bias"))
        self.declare_param("dt_bias", (H,), init="ones", decay=False, hf=hf.direct(f"{_M}.dt_bias"))
        self.declare_param("A_log", (H,), init="ones", decay=False, hf=hf.direct(f"{_M}.A_log"))
        self.declare_param("D", (H,), init="ones", decay=False, hf=hf.direct(f"{_M}.D"))
        self.declare_param("mixer_norm_weight", (inner,), init="ones", decay=False, hf=hf.direct(f"{_M}.norm.weight"))
        self.declare_param("out_weight", (d_model, inner), hf=hf.direct(f"{_M}.out_proj.weight"), quantizable=True)

    def mixer(self, h, position_ids):
        return F.torch_fn("mamba2_mixer", [h] + [self.p(n) for n in ("in_weight", "conv_weight", "conv_bias", "dt_bias", "A_log", "D", "mixer_norm_weight",
                                                                     "out_weight")], [("mamba_out", h.shape, "act")], **self.attrs)


class NemotronHAttentionBlock(_MixerBlock):
    def __init__(self, d_model, num_query_heads, num_kv_heads, head_size, eps=1e-5, **_):
        super().__init__(d_model, eps)
        self.Hq, self.Hkv, self.D = num_query_heads, num_kv_heads, head_size
        qd, kd = num_query_heads * head_size, num_kv_heads * head_size
        self.declare_param("qkv_weight", (qd + 2 * kd, d_model), quantizable=True,
                           hf=hf.fuse([f"{_M}.q_proj.weight", f"{_M}.k_proj.weight", f"{_M}.v_proj.weight"], sizes=[qd, kd, kd]),
                           lora_targets=[("q_proj", 0, qd), ("k_proj", qd, kd), ("v_proj", qd + kd, kd)])
        self.declare_param("out_weight", (d_model, qd), quantizable=True, hf=hf.direct(f"{_M}.o_proj.weight"), lora_targets=[("o_proj", 0, d_model)])

    def mixer(self, h, position_ids):
        qkv = F.matmul(h, self.p("qkv_weight"), name="qkv", role="qkv")
        att, _ = F.flash_attention(qkv, num_q_heads=self.Hq, num_kv_heads=self.Hkv, head_dim=self.D)  # no positional encoding in this family
        return F.matmul(att, self.p("out_weight"), name="att_out", role="out")


class NemotronHMoEBlock(_MixerBlock):
    def __init__(self, d_model, num_experts, num_experts_per_tok, moe_d_ff, shared_d_ff, n_group=1, topk_group=1, norm_topk_prob=True,
                 routed_scaling_factor=1.0, eps=1e-5, ep_size=1, **_):
        super().__init__(d_model, eps)
        self.E, self.K, self.ep_size = num_experts, num_experts_per_tok, ep_size
        self.attrs = dict(top_k=num_experts_per_tok, n_group=n_group, topk_group=topk_group, norm_topk_prob=norm_topk_prob,
                          routed_scaling_factor=routed_scaling_factor)
        self.declare_param("router_weight", (num_experts, d_model), hf=hf.direct(f"{_M}.gate.weight"))
        self.declare_param("router_score_bias", (num_experts,), init="zeros", decay=False, hf=hf.direct(f"{_M}.gate.e_score_correction_bias"))
        self.declare_param("experts_up", (num_experts, moe_d_ff, d_model), hf=hf.stack_experts([f"{_M}.experts.{{E}}.up_proj.weight"], num_experts))
        self.declare_param("experts_down", (num_experts, d_model, moe_d_ff), hf=hf.stack_experts([f"{_M}.experts.{{E}}.down_proj.weight"], num_experts))
        self.declare_param("shared_up_weight", (shared_d_ff, d_model), hf=hf.direct(f"{_M}.shared_experts.up_proj.weight"))
        self.declare_param("shared_down_weight", (d_model, shared_d_ff), hf=hf.direct(f"{_M}.shared_experts.down_proj.weight"))

    def mixer(self, h, position_ids):
        """Router as a PyTorch function; the experts run on the grouped GEMM path (permute -> up -> ReLU^2 -> down -> weighted
        un-permute, expert-parallel when ``ep_size`` > 1); the shared expert is two dense GEMMs."""
        lead = h.shape[:-1]
        tw, ti = F.torch_fn("sigmoid_group_router", [h, self.p("router_weight"), self.p("router_score_bias")],
                            [("topk_weights", lead + (self.K,), "fp32"), ("topk_index", lead + (self.K,), "int32")], **self.attrs)
        xp, plan = F.moe_permute(h, ti, num_experts=self.E, top_k=self.K)
        if self.ep_size > 1:
            xp, plan = F.ep_dispatch(xp, plan)
        u = F.moe_grouped_gemm(xp, self.p("experts_up"), plan, name="moe_up", role="experts_gate_up")
        a = F.torch_fn("relu2", [u], [("moe_relu2", u.shape, "act")])
        d = F.moe_grouped_gemm(a, self.p("experts_down"), plan, name="moe_down", role="experts_down")
        if self.ep_size > 1:
            d = F.ep_combine(d, plan)
        y = F.moe_unpermute(d, tw, plan, h.shape)
        su = F.matmul(h, self.p("shared_up_weight"), name="shared_up", role="shared_up")
        sa = F.torch_fn("relu2", [su], [("shared_relu2", su.shape, "act")])
        return F.add(y, F.matmul(sa, self.p("shared_down_weight"), name="shared_down", role="shared_down"), name="moe_plus_shared")

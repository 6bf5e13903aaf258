"""Mixture-of-experts feed-forward: router -> top-k -> permute -> [EP dispatch] -> grouped gate/up GEMM ->
SwiGLU -> grouped down GEMM -> [EP combine] -> weighted un-permute.

Parity: surogate/dsl/modules/moe.py:13-286 (MoEExpertsGated), :512 (MoESharedExpert).
"""
from __future__ import annotations

from .. import functional as F
from .. import hf
from ..nn import Module


class MoEExpertsGated(Module):
    def __init__(self, d_model: int, d_ff: int, num_experts: int, num_experts_per_tok: int = 8, norm_topk_prob: bool = True,
                 ep_size: int = 1, aux_loss_coef: float = 1e-3, z_loss_coef: float = 0.0, scoring: str = "softmax",
                 prefix: str = "model.layers.{L}.mlp", fused_checkpoint_experts: bool = False):
        """``fused_checkpoint_experts``: the checkpoint stores all experts of a layer as two 3-D tensors
        (``experts.gate_up_proj`` [E, 2F, C] with the gate rows first, ``experts.down_proj`` [E, C, F])."""
        super().__init__()
        self.E, self.K, self.ep_size = num_experts, num_experts_per_tok, ep_size
        self.norm_topk_prob, self.aux, self.z, self.scoring = norm_topk_prob, aux_loss_coef, z_loss_coef, scoring
        m = prefix
        self.declare_param("router_weight", (num_experts, d_model), hf=hf.direct(f"{m}.gate.weight"), decay=True)
        if fused_checkpoint_experts:
            gate_up_hf, down_hf = hf.transform(f"{m}.experts.gate_up_proj", fn="swap_row_halves"), hf.direct(f"{m}.experts.down_proj")
        else:
            gate_up_hf = hf.stack_experts([f"{m}.experts.{{E}}.up_proj.weight", f"{m}.experts.{{E}}.gate_proj.weight"], num_experts, sizes=[d_ff, d_ff])
            down_hf = hf.stack_experts([f"{m}.experts.{{E}}.down_proj.weight"], num_experts)
        self.declare_param("experts_gate_up", (num_experts, 2 * d_ff, d_model), quantizable=True, hf=gate_up_hf,
                           lora_targets=[("up_proj", 0, d_ff), ("gate_proj", d_ff, d_ff)])
        self.declare_param("experts_down", (num_experts, d_model, d_ff), quantizable=True, hf=down_hf, lora_targets=[("down_proj", 0, d_model)])

    def forward(self, x):
        tw, ti, aux = F.moe_router(x, self.p("router_weight"), top_k=self.K, norm_topk_prob=self.norm_topk_prob,
                                   aux_loss_coef=self.aux, z_loss_coef=self.z, scoring=self.scoring)
        xp, plan = F.moe_permute(x, ti, num_experts=self.E, top_k=self.K)
        if self.ep_size > 1:
            xp, plan = F.ep_dispatch(xp, plan)
        h = F.moe_grouped_gemm(xp, self.p("experts_gate_up"), plan, name="moe_gate_up", role="experts_gate_up")
        h = F.swiglu(h, name="moe_swiglu")
        h = F.moe_grouped_gemm(h, self.p("experts_down"), plan, name="moe_down", role="experts_down")
        if self.ep_size > 1:
            h = F.ep_combine(h, plan)
        y = F.moe_unpermute(h, tw, plan, x.shape)
        return y, aux


class MoESharedExpert(Module):
    """Dense SwiGLU expert applied to every token and added to the routed output."""

    def __init__(self, d_model: int, d_ff: int, prefix: str = "model.layers.{L}.mlp.shared_expert", gate_name: str = ""):
        """``gate_name``: checkpoint name of a [1, C] weight; when given the shared output is scaled by sigmoid(x . w) per token."""
        super().__init__()
        m = prefix
        self.gated = bool(gate_name)
        if self.gated:
            self.declare_param("shared_gate_weight", (1, d_model), hf=hf.direct(gate_name))
        self.declare_param("up_weight", (2 * d_ff, d_model), quantizable=True,
                           hf=hf.fuse([f"{m}.up_proj.weight", f"{m}.gate_proj.weight"], sizes=[d_ff, d_ff]))
        self.declare_param("down_weight", (d_model, d_ff), quantizable=True, hf=hf.direct(f"{m}.down_proj.weight"))

    def forward(self, x):
        up = F.matmul(x, self.p("up_weight"), name="shared_up", role="shared_up")
        y = F.matmul(F.swiglu(up, name="shared_swiglu"), self.p("down_weight"), name="shared_down", role="shared_down")
        if self.gated:
            y = F.torch_fn("sigmoid_gate_mul", [x, self.p("shared_gate_weight"), y], [("shared_gated", y.shape, "act")])
        return y

"""Embedding, LM head (fused with the loss), RMSNorm and plain Linear.

Parity: surogate/dsl/modules/embedding.py:12,102; rmsnorm.py:11-98.
"""
from __future__ import annotations

from .. import functional as F
from .. import hf
from ..nn import Module


class Embedding(Module):
    def __init__(self, vocab_size: int, d_model: int, hf_name: str = "model.embed_tokens.weight"):
        super().__init__()
        self.declare_param("weight", (vocab_size, d_model), hf=hf.direct(hf_name), decay=False)

    def forward(self, token_ids):
        return F.embedding(token_ids, self.p("weight"))


class LMHead(Module):
    """Projection to the vocabulary fused with cross-entropy; logits are produced and consumed chunk by chunk."""

    def __init__(self, vocab_size: int, d_model: int, tie_to: str | None = None, hf_name: str = "lm_head.weight", softcap: float = 0.0):
        super().__init__()
        self.tie_to = tie_to
        self.softcap = softcap
        mapping = hf.tied_to(hf_name, tie_to) if tie_to else hf.direct(hf_name)
        self.declare_param("weight", (vocab_size, d_model), hf=mapping, decay=True)

    def forward(self, x, targets):
        return F.fused_lm_head_loss(x, self.p("weight"), targets, softcap=self.softcap)


class RMSNorm(Module):
    """One-argument form: y = rmsnorm(x).  Two-argument form: residual += x ; y = rmsnorm(residual) in one op."""

    def __init__(self, d_model: int, eps: float = 1e-6, hf_name: str | None = None, out_name: str = "ln", res_name: str = "res",
                 zero_centered: bool = False):
        super().__init__()
        self.eps, self.out_name, self.res_name = eps, out_name, res_name
        # zero_centered: the checkpoint stores w - 1 (y = x_hat * (1 + w)); one is added on load and removed on export
        mapping = (hf.transform(hf_name, "plus_one") if zero_centered else hf.direct(hf_name)) if hf_name else None
        self.declare_param("weight", (d_model,), init="ones", decay=False, hf=mapping)

    def forward(self, a, b=None):
        if b is None:
            y, _ = F.rmsnorm(a, self.p("weight"), self.eps, name=self.out_name)
            return y
        res, y, _ = F.fused_residual_rmsnorm(a, b, self.p("weight"), self.eps, name=self.out_name, res_name=self.res_name)
        return res, y


class Linear(Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, hf_name: str | None = None, role: str = ""):
        super().__init__()
        self.role = role
        self.declare_param("weight", (out_features, in_features), hf=hf.direct(hf_name) if hf_name else None, quantizable=True)
        self.has_bias = bias
        if bias:
            self.declare_param("bias", (out_features,), init="zeros", decay=False,
                               hf=hf.direct(hf_name.replace(".weight", ".bias")) if hf_name else None)

    def forward(self, x):
        return F.matmul(x, self.p("weight"), self.p("bias") if self.has_bias else None, role=self.role)

"""Depth-wise causal 1-D convolution on channels-last activations, with its autograd function.

``causal_conv1d(x, w, bias, activation, seq_id)``: x ``[B, T, C]``, w ``[C, K]`` (K <= 4), bias ``[C]`` or None, activation ``None`` or
``"silu"``, seq_id int32 ``[B, T]`` or None (packed documents: taps do not cross a change of id).  On a GPU it runs the CUDA kernels of
``csrc/conv1d_kernels.cu`` (no transposes, one pass); elsewhere ``torch.nn.functional.conv1d``.  The PyTorch form is also the oracle of the
kernel tests.

Parity: the vendored causal-conv1d kernels the reference uses for Mamba-2 / gated delta-net / LFM2 layers.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F


def causal_conv1d_reference(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, activation: Optional[str] = None,
                            seq_id: Optional[torch.Tensor] = None) -> torch.Tensor:
    B, T, C = x.shape
    K = w.shape[1]
    if seq_id is None:
        y = F.conv1d(F.pad(x.transpose(1, 2), (K - 1, 0)), w.to(x.dtype).reshape(C, 1, K), None if bias is None else bias.to(x.dtype), groups=C).transpose(1, 2)
    else:
        y = x.new_zeros(B, T, C) if bias is None else bias.to(x.dtype).expand(B, T, C).clone()
        for k in range(K):
            shift = K - 1 - k
            xs = F.pad(x, (0, 0, shift, 0))[:, :T]
            ids = F.pad(seq_id, (shift, 0), value=-1)[:, :T]
            y = y + torch.where((ids == seq_id).unsqueeze(-1), xs * w[:, k].to(x.dtype), torch.zeros_like(xs))
    return F.silu(y) if activation == "silu" else y


class _CausalConv1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, silu: bool, seq_id):
        from . import ext

        e = ext()
        xc = x.contiguous()
        w32 = w.float().contiguous()
        b32 = None if bias is None else bias.float().contiguous()
        ctx.save_for_backward(xc, w32, b32 if b32 is not None else torch.empty(0, device=x.device), seq_id if seq_id is not None else torch.empty(0, device=x.device))
        ctx.silu, ctx.has_bias, ctx.has_ids, ctx.wdtype, ctx.bdtype = silu, bias is not None, seq_id is not None, w.dtype, None if bias is None else bias.dtype
        return e.causal_conv1d_fwd(xc, w32, b32, seq_id, silu)

    @staticmethod
    def backward(ctx, dy):
        from . import ext

        e = ext()
        x, w32, b32, ids = ctx.saved_tensors
        ids = ids if ctx.has_ids else None
        dz = dy.contiguous()
        if ctx.silu:   # fold the activation's derivative into the gradient of the pre-activation (one extra pass of the forward kernel)
            z = e.causal_conv1d_fwd(x, w32, b32 if ctx.has_bias else None, ids, False).float()
            sg = torch.sigmoid(z)
            dz = (dz.float() * sg * (1 + z * (1 - sg))).to(x.dtype)
        dx, dw, db = e.causal_conv1d_bwd(dz, x, w32, ids)
        return dx, dw.to(ctx.wdtype), (db.to(ctx.bdtype) if ctx.has_bias else None), None, None


def causal_conv1d(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, activation: Optional[str] = None,
                  seq_id: Optional[torch.Tensor] = None) -> torch.Tensor:
    ok = (x.is_cuda and x.dim() == 3 and x.dtype in (torch.bfloat16, torch.float32) and x.shape[-1] % 8 == 0 and 1 <= w.shape[1] <= 4
          and activation in (None, "silu"))
    if not ok:
        return causal_conv1d_reference(x, w, bias, activation, seq_id)
    return _CausalConv1d.apply(x, w, bias, activation == "silu", None if seq_id is None else seq_id.to(torch.int32).contiguous())

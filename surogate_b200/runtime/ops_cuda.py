"""CUDA backend: the IR ops implemented with the hand-written sm_100a kernels.

Subclasses the PyTorch reference backend and overrides the hot ops; anything not
overridden (rare, cold ops) runs the reference implementation on the GPU.  The
extension is mandatory here: constructing this backend without it raises, so a
GPU run can never silently fall back to library kernels.

GEMM conventions (see csrc/gemm_sm100.cu): ``gemm(a, b, d, a_mn, b_mn)`` computes
``d = op(a) @ op(b)^T`` where an operand flagged ``*_mn`` is stored
``[contraction, rows]``.  With that, forward / dgrad / wgrad all consume tensors
as they lie in memory:

* forward  y[M,N]  = x[M,K] . W[N,K]^T      -> gemm(x,  W,  a_mn=False, b_mn=False)
* dgrad    dx[M,K] = dy[M,N] . W[N,K]       -> gemm(dy, W,  a_mn=False, b_mn=True)
* wgrad    dW[N,K] = dy[M,N]^T . x[M,K]     -> gemm(dy, x,  a_mn=True,  b_mn=True)
"""
from __future__ import annotations

import math
from typing import Any, Optional

import torch

from ..ops import ext as _ext
from .ops_ref import IGNORE_INDEX, RefOps


class Fp8Tensor:
    """An FP8 payload with its per-tensor de-scale (1/scale) kept on the device."""

    __slots__ = ("data", "scale_inv", "hp")

    def __init__(self, data: torch.Tensor, scale_inv: torch.Tensor, hp: Optional[torch.Tensor] = None):
        self.data, self.scale_inv, self.hp = data, scale_inv, hp

    @property
    def shape(self):
        return self.data.shape

    @property
    def dtype(self):
        return torch.bfloat16

    @property
    def device(self):
        return self.data.device

    @property
    def is_cuda(self):
        return True

    def reshape(self, *shape):
        return Fp8Tensor(self.data.reshape(*shape), self.scale_inv, self.hp.reshape(*shape) if self.hp is not None else None)

    def dequantize(self) -> torch.Tensor:
        return (self.data.float() * self.scale_inv).to(torch.bfloat16)


def gemm(a, b, out=None, *, a_mn=False, b_mn=False, accumulate=False, alpha=1.0, scale_a=None, scale_b=None, amax_out=None,
         out_dtype=torch.bfloat16, tile_n=0):
    """Thin wrapper over the tcgen05 GEMM; allocates the output when not given."""
    ext = _ext()
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
        accumulate = False
    ext.gemm(a, b, out, a_mn, b_mn, accumulate, float(alpha), scale_a, scale_b, amax_out, 0, 0, tile_n)
    return out


class CudaOps(RefOps):
    name = "cuda"

    def __init__(self, lmhead_chunk_rows: int = 4096, attention: str = "auto"):
        super().__init__(lmhead_chunk_rows)
        self.ext = _ext()  # raises when the extension is unavailable
        self.attention_impl = attention

    # ------------------------------------------------------------------ embedding
    def embedding(self, ctx, op, token_ids, weight):
        if weight.dtype != torch.bfloat16:
            return super().embedding(ctx, op, token_ids, weight)
        return (self.ext.embedding_fwd(token_ids.contiguous(), weight),)

    def embedding_backward(self, ctx, op, d_x, token_ids):
        tgt, acc = ctx.grad_target(op.outputs[0])
        if tgt is None:
            return (None,)
        if not acc:
            tgt.zero_()
        self.ext.embedding_bwd(token_ids.contiguous(), d_x.contiguous(), tgt)
        return (None,)

    # ------------------------------------------------------------------ norms
    def rmsnorm(self, ctx, op, x, w):
        want8 = ctx.recipe is not None and ctx.recipe.wants_fp8_activation(ctx, op, 0)
        if want8:
            return ctx.recipe.norm_forward(ctx, op, self.ext, x, None, w)[1:]
        _, y, rstd, _ = self.ext.rmsnorm_fwd(x, None, w, op.attrs["eps"], True, None, None, False)
        return y, rstd

    def fused_residual_rmsnorm(self, ctx, op, residual, x, w):
        want8 = ctx.recipe is not None and ctx.recipe.wants_fp8_activation(ctx, op, 1)
        if want8:
            return ctx.recipe.norm_forward(ctx, op, self.ext, x, residual, w)
        res, y, rstd, _ = self.ext.rmsnorm_fwd(x, residual, w, op.attrs["eps"], True, None, None, False)
        return res, y, rstd

    def rmsnorm_backward(self, ctx, op, dy, x, w, rstd, d_res):
        dx, dw = self.ext.rmsnorm_bwd(dy.contiguous(), x, w, rstd, d_res)
        return dx, dw

    # ------------------------------------------------------------------ matmul
    def matmul(self, ctx, op, x, w, bias):
        y = ctx.recipe.forward_matmul(ctx, op, x, w, bias) if ctx.recipe is not None else None
        if y is None:
            K = x.shape[-1]
            y = gemm(x.reshape(-1, K), w).reshape(*x.shape[:-1], w.shape[0])
            if bias is not None:
                y += bias
        if ctx.lora is not None:
            y = ctx.lora.forward(ctx, op, x, y)
        return (y,)

    def matmul_backward(self, ctx, op, dy, x, w):
        K, N = x.shape[-1], dy.shape[-1]
        dy2 = dy.reshape(-1, N)
        x2 = x.reshape(-1, K)
        if ctx.lora is not None:
            extra_dx = ctx.lora.backward(ctx, op, dy2, x2)
        else:
            extra_dx = None
        r = ctx.recipe.backward_matmul(ctx, op, dy2, x2, w) if ctx.recipe is not None else None
        if r is not None:
            dx = r[0]
        else:
            dx = gemm(dy2, w, a_mn=False, b_mn=True)
            tgt, acc = ctx.grad_target(op.outputs[1])
            if tgt is not None:
                gemm(dy2, x2, tgt, a_mn=True, b_mn=True, accumulate=acc)
        if extra_dx is not None:
            dx += extra_dx
        db = dy2.float().sum(0) if op.outputs[2] is not None else None
        return dx.reshape(x.shape), None, db

    # ------------------------------------------------------------------ qk-norm + rope
    def qkv_qk_norm_rope(self, ctx, op, qkv, qw, kw, pos):
        a = op.attrs
        if a["head_dim"] != 128 or a["rotary_dim"] != 128 or qkv.dtype != torch.bfloat16:
            return super().qkv_qk_norm_rope(ctx, op, qkv, qw, kw, pos)
        out, q_rstd, k_rstd = self.ext.qk_norm_rope_fwd(qkv, qw, kw, pos.contiguous(), a["num_q_heads"], a["num_kv_heads"], 128, a["eps"],
                                                        a["rope_theta"])
        return out, (q_rstd if qw is not None else None), (k_rstd if qw is not None else None)

    def qkv_qk_norm_rope_backward(self, ctx, op, dy, qkv, qw, kw, q_rstd, k_rstd, pos):
        a = op.attrs
        if a["head_dim"] != 128 or a["rotary_dim"] != 128 or qkv.dtype != torch.bfloat16:
            return super().qkv_qk_norm_rope_backward(ctx, op, dy, qkv, qw, kw, q_rstd, k_rstd, pos)
        dx, dqw, dkw = self.ext.qk_norm_rope_bwd(dy.contiguous(), qkv, qw, kw, q_rstd, k_rstd, pos.contiguous(), a["num_q_heads"],
                                                 a["num_kv_heads"], 128, a["eps"], a["rope_theta"])
        return dx, (dqw if qw is not None else None), (dkw if qw is not None else None)

    # ------------------------------------------------------------------ swiglu
    def swiglu(self, ctx, op, x):
        if ctx.recipe is not None and ctx.recipe.wants_fp8_activation(ctx, op, 0):
            return (ctx.recipe.swiglu_forward(ctx, op, self.ext, x),)
        return (self.ext.swiglu_fwd(x, True, None, None, False)[0],)

    def swiglu_backward(self, ctx, op, dy, x):
        return (self.ext.swiglu_bwd(dy.contiguous(), x),)

    # ------------------------------------------------------------------ attention
    def flash_attention(self, ctx, op, qkv):
        from ..ops import attention as att_ops

        if att_ops.native_supported(op.attrs, qkv, ctx) and self.attention_impl in ("auto", "native"):
            return att_ops.forward(self.ext, op.attrs, qkv, ctx)
        return super().flash_attention(ctx, op, qkv)

    def flash_attention_backward(self, ctx, op, d_att, qkv, att, lse):
        from ..ops import attention as att_ops

        if torch.is_tensor(lse):
            return att_ops.backward(self.ext, op.attrs, d_att, qkv, att, lse, ctx)
        return super().flash_attention_backward(ctx, op, d_att, qkv, att, lse)

    # ------------------------------------------------------------------ LM head + loss
    def fused_lm_head_loss(self, ctx, op, x, w, targets):
        """Chunked over rows: logits chunk by GEMM (bf16), cross-entropy forward+backward in place, then the
        dgrad / wgrad GEMMs consume the in-place d_logits.  The full [tokens, vocab] matrix never exists."""
        if isinstance(x, Fp8Tensor):
            x = x.hp if x.hp is not None else x.dequantize()
        C = x.shape[-1]
        V = w.shape[0]
        x2 = x.reshape(-1, C)
        t = targets.reshape(-1).contiguous()
        n = x2.shape[0]
        train = ctx.training
        rows = min(self.lmhead_chunk_rows, n)
        logits = torch.empty(rows, V, dtype=torch.bfloat16, device=x.device)
        losses = torch.empty(n, dtype=torch.float32, device=x.device)
        dx = torch.empty_like(x2) if train else None
        tgt = None
        if train:
            tgt, acc = ctx.grad_target("grad::" + op.inputs[1])
        scale_t = ctx.loss_scale if torch.is_tensor(ctx.loss_scale) else None
        scale_h = 1.0 if scale_t is not None else float(ctx.loss_scale)
        for s in range(0, n, rows):
            e = min(s + rows, n)
            lg = logits[: e - s]
            gemm(x2[s:e], w, lg)
            losses[s:e] = self.ext.cross_entropy_fwd_bwd(lg, t[s:e], scale_t, scale_h, train)
            if train:
                gemm(lg, w, dx[s:e], a_mn=False, b_mn=True)
                if tgt is not None:
                    gemm(lg, x2[s:e], tgt, a_mn=True, b_mn=True, accumulate=acc)
                    acc = True
        if train:
            ctx.stash[op.outputs[0]] = dx.reshape(x.shape)
        return (losses.sum(),)


def make_backend(device: torch.device, kind: str = "auto", **kw):
    """``cuda`` = hand-written kernels (required on a GPU unless ``ref`` is asked for), ``ref`` = PyTorch reference."""
    if kind == "auto":
        kind = "cuda" if device.type == "cuda" else "ref"
    if kind == "cuda":
        return CudaOps(**kw)
    kw.pop("attention", None)
    return RefOps(**kw)

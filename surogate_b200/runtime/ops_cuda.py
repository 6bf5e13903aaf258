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
        self.stack = None  # runtime.memory.DeviceStack: transients of the LM-head chunk loop (SUROGATE_DEVICE_STACK=0 switches it off)

    def _transient_stack(self, device):
        import os

        if self.stack is None and os.environ.get("SUROGATE_DEVICE_STACK", "1") != "0":
            try:
                from .memory import DeviceStack

                self.stack = DeviceStack(device, name="transients")
            except Exception:  # noqa: BLE001 - host runtime not built: buffers come from the caching allocator
                self.stack = False
        return self.stack or None

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
        elif isinstance(dy2, Fp8Tensor):
            raise RuntimeError("an FP8 gradient reached a matmul whose backward is not FP8")
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
    @staticmethod
    def _multi_axis(ctx, a) -> bool:
        """A batch with image / video tokens carries (t, h, w) positions."""
        return bool(a.get("mrope_section")) and ctx.extras.get("mrope_position_ids") is not None

    def _rope_positions(self, ctx, a, pos):
        """(position tensor, sec_h, sec_w) for the kernel: three rows and the section sizes when the batch carries (t, h, w)
        positions and the op is a multi-axis one, else the plain [B, T] positions."""
        if self._multi_axis(ctx, a):
            sec = a["mrope_section"]
            return ctx.extras["mrope_position_ids"].to(torch.int32).contiguous(), int(sec[1]), int(sec[2])
        return pos.contiguous(), 0, 0

    def _rope_kernel_ok(self, a, qkv) -> bool:
        return a["head_dim"] == 128 and a["rotary_dim"] == 128 and qkv.dtype == torch.bfloat16 and not a.get("rope_scaling")

    def qkv_qk_norm_rope(self, ctx, op, qkv, qw, kw, pos):
        a = op.attrs
        if not self._rope_kernel_ok(a, qkv):
            return super().qkv_qk_norm_rope(ctx, op, qkv, qw, kw, pos)
        p, sh, sw = self._rope_positions(ctx, a, pos)
        out, q_rstd, k_rstd = self.ext.qk_norm_rope_fwd(qkv, qw, kw, p, a["num_q_heads"], a["num_kv_heads"], 128, a["eps"], a["rope_theta"], sh, sw)
        return out, (q_rstd if qw is not None else None), (k_rstd if qw is not None else None)

    def qkv_qk_norm_rope_backward(self, ctx, op, dy, qkv, qw, kw, q_rstd, k_rstd, pos):
        a = op.attrs
        if not self._rope_kernel_ok(a, qkv):
            return super().qkv_qk_norm_rope_backward(ctx, op, dy, qkv, qw, kw, q_rstd, k_rstd, pos)
        p, sh, sw = self._rope_positions(ctx, a, pos)
        dx, dqw, dkw = self.ext.qk_norm_rope_bwd(dy.contiguous(), qkv, qw, kw, q_rstd, k_rstd, p, a["num_q_heads"], a["num_kv_heads"], 128, a["eps"],
                                                 a["rope_theta"], sh, sw)
        return dx, (dqw if qw is not None else None), (dkw if qw is not None else None)

    # ------------------------------------------------------------------ swiglu
    def swiglu(self, ctx, op, x):
        if ctx.recipe is not None and ctx.recipe.wants_fp8_activation(ctx, op, 0):
            return (ctx.recipe.swiglu_forward(ctx, op, self.ext, x),)
        used = getattr(x, "_sg_rows", None)   # expert rows in a worst-case sized buffer: only the rows in use are processed
        y = self.ext.swiglu_fwd(x, True, None, None, False, used)[0]
        if used is not None:
            y._sg_rows = used
        return (y,)

    def swiglu_backward(self, ctx, op, dy, x):
        if ctx.recipe is not None and hasattr(ctx.recipe, "swiglu_backward_fp8"):
            d8 = ctx.recipe.swiglu_backward_fp8(ctx, op, self.ext, dy, x)
            if d8 is not None:
                return (d8,)
        used = getattr(x, "_sg_rows", None)
        if used is None:
            used = getattr(dy, "_sg_rows", None)
        dx = self.ext.swiglu_bwd(dy.contiguous(), x, used)
        if used is not None:
            dx._sg_rows = used
        return (dx,)

    # ------------------------------------------------------------------ tiled MLP (long context): same tiles on the tcgen05 GEMM + SwiGLU kernels
    def tiled_mlp(self, ctx, op, x, up_w, down_w):
        if x.dtype != torch.bfloat16 or up_w.dtype != torch.bfloat16:
            return super().tiled_mlp(ctx, op, x, up_w, down_w)
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        rows = max(128, int(op.attrs["tile_rows"]) // 128 * 128)
        y = torch.empty(x2.shape[0], down_w.shape[0], dtype=x.dtype, device=x.device)
        for s in range(0, x2.shape[0], rows):
            a = self.ext.swiglu_fwd(gemm(x2[s:s + rows], up_w), True, None, None, False)[0]
            gemm(a, down_w, y[s:s + rows])
        return (y.reshape(*x.shape[:-1], down_w.shape[0]),)

    def tiled_mlp_backward(self, ctx, op, dy, x, up_w, down_w):
        if x.dtype != torch.bfloat16 or up_w.dtype != torch.bfloat16:
            return super().tiled_mlp_backward(ctx, op, dy, x, up_w, down_w)
        C = x.shape[-1]
        x2, dy2 = x.reshape(-1, C), dy.reshape(-1, dy.shape[-1]).contiguous()
        rows = max(128, int(op.attrs["tile_rows"]) // 128 * 128)
        dx = torch.empty_like(x2)
        g_up, acc_up = ctx.grad_target(op.outputs[1])
        g_down, acc_down = ctx.grad_target(op.outputs[2])
        for s in range(0, x2.shape[0], rows):
            xc, dyc = x2[s:s + rows], dy2[s:s + rows]
            u = gemm(xc, up_w)
            a = self.ext.swiglu_fwd(u, True, None, None, False)[0]
            da = gemm(dyc, down_w, b_mn=True)
            du = self.ext.swiglu_bwd(da, u)
            gemm(du, up_w, dx[s:s + rows], b_mn=True)
            if g_down is not None:
                gemm(dyc, a, g_down, a_mn=True, b_mn=True, accumulate=acc_down or s > 0)
            if g_up is not None:
                gemm(du, xc, g_up, a_mn=True, b_mn=True, accumulate=acc_up or s > 0)
        return dx.reshape(x.shape), None, None

    # ------------------------------------------------------------------ attention
    # ------------------------------------------------------------------ attention of a sequence chunk against its key/value prefix
    # The tcgen05 kernels take equal query and key lengths.  A chunk's queries against all keys up to its end are therefore run
    # as causal attention over prefix + chunk with zero queries in the prefix rows: those rows cost compute but nothing else
    # (their output is dropped; in backward their dO is zero, so they add nothing to dK / dV).
    def _chunk_native_ok(self, ctx, a, qkv) -> bool:
        cs = ctx.chunk
        return (self.attention_impl in ("auto", "native") and hasattr(self.ext, "flash_attn_fwd") and a["head_dim"] == 128 and a.get("causal", True)
                and not a.get("window", 0) and qkv.dtype == torch.bfloat16 and ctx.doc_ids is None and cs.chunk_len % 128 == 0 and qkv.shape[1] == cs.chunk_len)

    def _chunk_packed(self, ctx, a, q):
        cs, L = ctx.chunk, ctx.layer
        Hq, Hkv, D = a["num_q_heads"], a["num_kv_heads"], a["head_dim"]
        B, Tc = q.shape[:2]
        n = cs.index * cs.chunk_len
        full = torch.zeros(B, n + Tc, Hq + 2 * Hkv, D, dtype=torch.bfloat16, device=q.device)
        full[:, :, Hq:Hq + Hkv] = cs.k[L][:, :n + Tc]
        full[:, :, Hq + Hkv:] = cs.v[L][:, :n + Tc]
        full[:, n:, :Hq] = q
        return full.view(B, n + Tc, (Hq + 2 * Hkv) * D), n

    def _chunk_attention_native(self, ctx, op, qkv):
        a = op.attrs
        Hq, Hkv, D = a["num_q_heads"], a["num_kv_heads"], a["head_dim"]
        scale = a.get("softmax_scale") or 1.0 / math.sqrt(D)
        q, k, v = self._split_heads(qkv, a)
        ctx.chunk.store_kv(ctx.layer, k, v)
        full, n = self._chunk_packed(ctx, a, q)
        att, lse = self.ext.flash_attn_fwd(full, Hq, Hkv, float(scale))
        return att[:, n:].contiguous(), lse[:, n:].contiguous()

    def _chunk_attention_native_backward(self, ctx, op, d_att, qkv, att, lse):
        a, cs = op.attrs, ctx.chunk
        Hq, Hkv, D = a["num_q_heads"], a["num_kv_heads"], a["head_dim"]
        scale = a.get("softmax_scale") or 1.0 / math.sqrt(D)
        B, Tc = qkv.shape[:2]
        q, _, _ = self._split_heads(qkv, a)
        full, n = self._chunk_packed(ctx, a, q)
        att_full, lse_full = self.ext.flash_attn_fwd(full, Hq, Hkv, float(scale))  # outputs / log-sum-exp of the prefix rows are needed by the kernel
        d_full = torch.zeros_like(att_full)
        d_full[:, n:] = d_att
        dfull = self.ext.flash_attn_bwd(d_full, full, att_full, lse_full, Hq, Hkv, float(scale)).view(B, n + Tc, Hq + 2 * Hkv, D)
        dk_acc, dv_acc = cs.grad_buffers(ctx.layer)
        dk_acc[:, :n + Tc] += dfull[:, :, Hq:Hq + Hkv].float()
        dv_acc[:, :n + Tc] += dfull[:, :, Hq + Hkv:].float()
        own = slice(n, n + Tc)  # by now these rows also hold what the later chunks contributed
        out = torch.cat([dfull[:, n:, :Hq].float(), dk_acc[:, own], dv_acc[:, own]], dim=2)
        return (out.reshape(qkv.shape).to(qkv.dtype),)

    def flash_attention(self, ctx, op, qkv):
        from ..ops import attention as att_ops

        if ctx.chunk is not None and self._chunk_native_ok(ctx, op.attrs, qkv):
            return self._chunk_attention_native(ctx, op, qkv)

        if ctx.chunk is None and att_ops.native_supported(op.attrs, qkv, ctx) and self.attention_impl in ("auto", "native"):
            return att_ops.forward(self.ext, op.attrs, qkv, ctx)
        return super().flash_attention(ctx, op, qkv)  # incl. chunked sequences: blockwise PyTorch attention against the key/value prefix

    def flash_attention_backward(self, ctx, op, d_att, qkv, att, lse):
        from ..ops import attention as att_ops

        if ctx.chunk is not None and self._chunk_native_ok(ctx, op.attrs, qkv):
            return self._chunk_attention_native_backward(ctx, op, d_att, qkv, att, lse)
        if torch.is_tensor(lse) and ctx.chunk is None:
            return att_ops.backward(self.ext, op.attrs, d_att, qkv, att, lse, ctx)
        return super().flash_attention_backward(ctx, op, d_att, qkv, att, lse)

    # ------------------------------------------------------------------ LM head + loss
    def fused_lm_head_loss(self, ctx, op, x, w, targets):
        """Chunked over rows: logits chunk by GEMM (bf16), cross-entropy forward+backward in place, then the
        dgrad / wgrad GEMMs consume the in-place d_logits.  The full [tokens, vocab] matrix never exists."""
        dropped = self._drop_ignored_rows(ctx, op, x, w, targets)
        if dropped is not None:
            return dropped
        if isinstance(x, Fp8Tensor):
            x = x.hp if x.hp is not None else x.dequantize()
        C = x.shape[-1]
        V = w.shape[0]
        x2 = x.reshape(-1, C)
        t = targets.reshape(-1).contiguous()
        n = x2.shape[0]
        train = ctx.training
        rows = min(self.lmhead_chunk_rows, n)
        stack = self._transient_stack(x.device)
        if stack is not None and stack.fits(rows * V * 2):
            with stack.frame():  # the chunk buffer has the same address every step (also under graph replay) and never touches the allocator
                return self._lm_head_chunks(ctx, op, x, w, x2, t, n, rows, stack.alloc((rows, V), torch.bfloat16, "lm_head.logits"))
        return self._lm_head_chunks(ctx, op, x, w, x2, t, n, rows, torch.empty(rows, V, dtype=torch.bfloat16, device=x.device))

    def _lm_head_chunks(self, ctx, op, x, w, x2, t, n, rows, logits):
        C, V = x2.shape[-1], w.shape[0]
        train = ctx.training
        losses = torch.empty(n, dtype=torch.float32, device=x.device)
        dx = torch.empty_like(x2) if train else None
        tgt = None
        if train:
            tgt, acc = ctx.grad_target("grad::" + op.inputs[1])
        scale_t = ctx.loss_scale if torch.is_tensor(ctx.loss_scale) else None
        scale_h = 1.0 if scale_t is not None else float(ctx.loss_scale)
        rw = ctx.row_weights.reshape(-1).float().contiguous() if ctx.row_weights is not None else None
        kd = ctx.kd
        kd_idx = kd["idx"].reshape(n, -1).to(torch.int32).contiguous() if kd else None
        kd_logp = kd["logp"].reshape(n, -1).float().contiguous() if kd else None
        kd_losses = torch.zeros(n, dtype=torch.float32, device=x.device) if kd else None
        if kd and kd.get("ce_weight", 1.0) != 1.0:  # total = ce_weight * CE + weight * KD
            cw = torch.full((n,), float(kd["ce_weight"]), dtype=torch.float32, device=x.device)
            rw = cw if rw is None else rw * cw
        # FP8 LM head (FP8 recipe, plain cross-entropy): x and W in E4M3, d_logits in E5M2 with a scale known in advance
        # (|softmax - onehot| <= 1, times the loss scale), so all three GEMMs of the head run at FP8 rate.
        fp8 = (getattr(ctx.recipe, "fp8_lm_head", False) and rw is None and kd is None and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
               and C % 16 == 0 and V % 16 == 0)
        if fp8:
            x8, x_inv = ctx.recipe.quantize_now(self.ext, x2)
            w8, w_inv = ctx.recipe.lm_head_weight(self.ext, w)
            if train:
                ls = scale_t.reshape(1).float() * scale_h if scale_t is not None else torch.full((1,), scale_h, dtype=torch.float32, device=x.device)
                d_scale = (57344.0 * 0.5) / ls.clamp_min(1e-30)
                d_inv = 1.0 / d_scale
        for s in range(0, n, rows):
            e = min(s + rows, n)
            lg = logits[: e - s]
            if fp8:
                gemm(x8[s:e], w8, lg, scale_a=x_inv, scale_b=w_inv)
            else:
                gemm(x2[s:e], w, lg)
            losses[s:e] = self.ext.cross_entropy_fwd_bwd(lg, t[s:e], scale_t, scale_h, train, rw[s:e] if rw is not None else None,
                                                         kd_idx[s:e] if kd else None, kd_logp[s:e] if kd else None, float(kd["weight"]) if kd else 0.0,
                                                         kd_losses[s:e] if kd else None)
            if train and fp8:
                d8 = self.ext.quantize_fp8(lg, d_scale, None, True)
                gemm(d8, w8, dx[s:e], a_mn=False, b_mn=True, scale_a=d_inv, scale_b=w_inv)
                if tgt is not None:
                    gemm(d8, x8[s:e], tgt, a_mn=True, b_mn=True, accumulate=acc, scale_a=d_inv, scale_b=x_inv)
                    acc = True
            elif train:
                gemm(lg, w, dx[s:e], a_mn=False, b_mn=True)
                if tgt is not None:
                    gemm(lg, x2[s:e], tgt, a_mn=True, b_mn=True, accumulate=acc)
                    acc = True
        if train:
            ctx.stash[op.outputs[0]] = dx.reshape(x.shape)
        if ctx.want_token_losses:
            ctx.stash["token_losses"] = losses
            if kd:
                ctx.stash["token_kd"] = kd_losses
        total = losses.sum()
        if kd:  # reported loss = ce_weight * CE + weight * KD (the gradient above already carries both)
            total = float(kd.get("ce_weight", 1.0)) * total + float(kd["weight"]) * kd_losses.sum()
        return (total,)


class CudaMoEPlan:
    """Device-side routing plan: padded per-expert row ranges and the row each (token, k) copy landed on."""

    def __init__(self, row_map, offsets, counts, capacity, num_tokens, top_k, num_experts, x_shape):
        self.row_map, self.offsets, self.counts, self.capacity = row_map, offsets, counts, capacity
        self.num_tokens, self.top_k, self.num_experts, self.x_shape = num_tokens, top_k, num_experts, x_shape
        self.local = None
        self.ep = None


def _moe_mixin():
    """MoE ops of the CUDA backend (kept together; attached to CudaOps below)."""

    def moe_router(self, ctx, op, x, rw):
        a = op.attrs
        E, K = a["num_experts"], a["top_k"]
        if a["scoring"] != "softmax" or x.dtype != torch.bfloat16 or E > 256:
            return RefOps.moe_router(self, ctx, op, x, rw)
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        N = x2.shape[0]
        logits = gemm(x2, rw, out_dtype=torch.float32)
        counts = torch.zeros(E, dtype=torch.int32, device=x.device)
        psum = torch.zeros(E, dtype=torch.float32, device=x.device)
        lse_sq = torch.zeros(1, dtype=torch.float32, device=x.device) if a.get("z_loss_coef", 0.0) else None
        tw, ti, _ = self.ext.moe_softmax_topk(logits, K, bool(a["norm_topk_prob"]), counts, psum, lse_sq, False)
        aux = a["aux_loss_coef"] * E * ((counts.float() / N) * (psum / N)).sum()
        if lse_sq is not None:
            aux = aux + a["z_loss_coef"] * lse_sq[0] / N
        ctx.stash[("moe_counts", ctx.layer, ctx.phase)] = counts
        ctx.record_moe_stats(counts.float(), (psum / N).unsqueeze(0))
        lead = x.shape[:-1]
        return tw.reshape(*lead, K), ti.reshape(*lead, K), aux

    def moe_router_backward(self, ctx, op, d_tw, d_aux, x, rw, tw, ti):
        a = op.attrs
        if a["scoring"] != "softmax" or x.dtype != torch.bfloat16 or a["num_experts"] > 256:
            return RefOps.moe_router_backward(self, ctx, op, d_tw, d_aux, x, rw, tw, ti)
        E, K = a["num_experts"], a["top_k"]
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        N = x2.shape[0]
        logits = gemm(x2, rw, out_dtype=torch.float32)   # recomputed: [N, E] fp32 is not kept from forward
        til = ti.reshape(N, K).contiguous()
        counts = da = None
        if d_aux is not None:
            da = d_aux if torch.is_tensor(d_aux) else torch.tensor(float(d_aux), dtype=torch.float32, device=x.device)
            da = da.to(torch.float32).reshape(1).contiguous()
            flat = til.reshape(-1).long()
            counts = torch.zeros(E, dtype=torch.int32, device=x.device).scatter_add_(0, flat, torch.ones_like(flat, dtype=torch.int32))  # no host sync
        g = d_tw.reshape(N, K).float().contiguous() if d_tw is not None else None
        # softmax, top-k selection gradient, auxiliary- and z-loss terms and the softmax Jacobian in one kernel (one warp per token)
        dl = self.ext.moe_router_bwd(logits, til, g, counts, da, bool(a["norm_topk_prob"]), float(a["aux_loss_coef"]), float(a.get("z_loss_coef", 0.0)))
        dx = gemm(dl, rw, b_mn=True).reshape(x.shape)          # [N,E] . [E,C]
        drw = gemm(dl, x2, a_mn=True, b_mn=True, out_dtype=torch.float32)   # [E,N] . [N,C]
        return dx, drw

    def moe_permute(self, ctx, op, x, ti):
        a = op.attrs
        E, K = a["num_experts"], a["top_k"]
        if x.dtype != torch.bfloat16 or E > 256:
            return RefOps.moe_permute(self, ctx, op, x, ti)
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        N = x2.shape[0]
        counts = ctx.stash.pop(("moe_counts", ctx.layer, ctx.phase), None)
        if counts is None:
            counts = torch.bincount(ti.reshape(-1).long(), minlength=E).to(torch.int32)
        if ctx.ep is not None:  # expert parallel: the dispatch kernel permutes while it sends; nothing moves here
            from ..parallel.ep import PrePlan

            ti_p, counts_p = ctx.ep.place(ctx.layer, ti.reshape(N, K).contiguous(), counts)  # least-loaded placement: expert id -> (rank, slot)
            return x2, PrePlan(ti_p, counts_p, N, K, E, tuple(x.shape))
        cap = N * K + E * 128                      # exact upper bound of the padded row count: no host read of the routing
        cap = (cap + 127) // 128 * 128
        offsets = torch.empty(E + 1, dtype=torch.int32, device=x.device)
        cursors = torch.empty(E, dtype=torch.int32, device=x.device)
        self.ext.moe_offsets(counts, offsets, cursors, cap, self.ext.error_flag_tensor())
        row_map = torch.empty(N * K, dtype=torch.int32, device=x.device)
        xp = torch.zeros(cap, C, dtype=x.dtype, device=x.device)   # pad rows must be zero (they enter the wgrad contraction)
        self.ext.moe_permute(x2, ti.reshape(N, K).contiguous(), offsets, cursors, row_map, xp, 0, E)
        return xp, CudaMoEPlan(row_map, offsets, counts, cap, N, K, E, tuple(x.shape))

    def moe_permute_backward(self, ctx, op, d_xp, plan):
        plan = getattr(plan, "ep_plan", None) or plan  # under EP the permutation happened inside the dispatch kernel
        if getattr(plan, "ep", None) is True:
            return (ctx.ep.combine(ctx, d_xp, None, plan, backward=True),)
        plan = plan.local or plan
        if not isinstance(plan, CudaMoEPlan):
            return RefOps.moe_permute_backward(self, ctx, op, d_xp, plan)
        dx = self.ext.moe_unpermute(d_xp.contiguous(), None, plan.row_map, plan.num_tokens, plan.top_k)
        return (dx.reshape(plan.x_shape),)

    def moe_grouped_gemm(self, ctx, op, x, w, plan):
        if not hasattr(plan, "offsets") or not hasattr(plan, "capacity"):
            return RefOps.moe_grouped_gemm(self, ctx, op, x, w, plan)
        r = ctx.recipe.forward_grouped(ctx, op, x, w, plan) if ctx.recipe is not None and hasattr(ctx.recipe, "forward_grouped") else None
        if r is not None:
            if ctx.lora is not None:
                r = ctx.lora.forward_grouped(ctx, op, x, r, plan)
            return (r,)
        used = getattr(x, "_sg_rows", None)
        # every row of a group (padding included) is written by the GEMM; rows behind the last group are never read into a result,
        # so a buffer sized for the worst case (expert parallel) is not cleared, only tagged with the row count in use
        y = (torch.empty if used is not None else torch.zeros)(x.shape[0], w.shape[1], dtype=x.dtype, device=x.device)
        self.ext.gemm_grouped(x, w, y, plan.offsets, 1, False, False, 1.0, None, None, self.ext.error_flag_tensor())
        if used is not None:
            y._sg_rows = used
        if ctx.lora is not None:
            y = ctx.lora.forward_grouped(ctx, op, x, y, plan)
        return (y,)

    def _expert_lora_backward(self, ctx, op, dy, x, plan, dx):
        extra = ctx.lora.backward_grouped(ctx, op, dy, x, plan) if ctx.lora is not None else None
        if extra is not None:
            used = getattr(dx, "_sg_rows", None)
            dx = dx + extra
            if used is not None:
                dx._sg_rows = used
        return dx

    def moe_grouped_gemm_backward(self, ctx, op, dy, x, w, plan):
        if not hasattr(plan, "offsets") or not hasattr(plan, "capacity"):
            return RefOps.moe_grouped_gemm_backward(self, ctx, op, dy, x, w, plan)
        r = ctx.recipe.backward_grouped(ctx, op, dy, x, w, plan) if ctx.recipe is not None and hasattr(ctx.recipe, "backward_grouped") else None
        if r is not None:
            return self._expert_lora_backward(ctx, op, dy, x, plan, r), None
        err = self.ext.error_flag_tensor()
        dy = dy.contiguous()
        used = getattr(dy, "_sg_rows", None)
        if used is None:
            used = getattr(x, "_sg_rows", None)
        dx = (torch.empty_like if used is not None else torch.zeros_like)(x)
        self.ext.gemm_grouped(dy, w, dx, plan.offsets, 1, True, False, 1.0, None, None, err)     # dy [R,N] . W[g] [N,K]
        if used is not None:
            dx._sg_rows = used
        tgt, acc = ctx.grad_target(op.outputs[1])
        if tgt is not None:
            # dW[g] (+)= dy_g^T . x_g ; groups without rows schedule no tiles, so their slices are cleared here (only theirs)
            self.ext.gemm_grouped(dy, x, tgt, plan.offsets, 2, True, acc, 1.0, None, None, err)
            if not acc:
                self.ext.zero_empty_groups(tgt, plan.offsets)
        return self._expert_lora_backward(ctx, op, dy, x, plan, dx), None

    def moe_unpermute(self, ctx, op, yp, tw, plan):
        if getattr(plan, "ep", None) is True:
            return (ctx.ep.combine(ctx, yp, tw, plan),)
        plan = plan.local or plan
        if not isinstance(plan, CudaMoEPlan):
            return RefOps.moe_unpermute(self, ctx, op, yp, tw, plan)
        y = self.ext.moe_unpermute(yp, tw.reshape(-1, plan.top_k).contiguous(), plan.row_map, plan.num_tokens, plan.top_k)
        return (y.reshape(plan.x_shape),)

    def moe_unpermute_backward(self, ctx, op, dy, yp, tw, plan):
        if getattr(plan, "ep", None) is True:
            return ctx.ep.combine_backward(ctx, dy, tw, plan)
        plan = plan.local or plan
        if not isinstance(plan, CudaMoEPlan):
            return RefOps.moe_unpermute_backward(self, ctx, op, dy, yp, tw, plan)
        d_yp, d_tw = self.ext.moe_unpermute_bwd(dy.reshape(plan.num_tokens, -1).contiguous(), yp, tw.reshape(-1, plan.top_k).contiguous(), plan.row_map)
        return d_yp, d_tw.reshape(tw.shape)

    def ep_dispatch(self, ctx, op, xp, plan):
        return ctx.ep.dispatch(ctx, xp, plan)

    def ep_combine(self, ctx, op, y, plan):
        # forward: expert outputs become pullable; as the backward of ep_dispatch: the experts' d_x become pullable
        return (ctx.ep.publish_outputs(ctx, y, plan, backward=bool(op.attrs.get("backward", False))),)

    def ep_dispatch_backward(self, ctx, op, dy, plan):
        return (dy,)  # combine_backward already delivered d_yp to the experts' owner

    for f in (ep_dispatch, ep_combine, ep_dispatch_backward):
        setattr(CudaOps, f.__name__, f)

    for f in (moe_router, moe_router_backward, moe_permute, moe_permute_backward, moe_grouped_gemm, moe_grouped_gemm_backward, moe_unpermute,
              moe_unpermute_backward, _expert_lora_backward):
        setattr(CudaOps, f.__name__, f)


_moe_mixin()


def make_backend(device: torch.device, kind: str = "auto", **kw):
    """``cuda`` = hand-written kernels (required on a GPU unless ``ref`` is asked for), ``ref`` = PyTorch reference."""
    if kind == "auto":
        kind = "cuda" if device.type == "cuda" else "ref"
    if kind == "cuda":
        return CudaOps(**kw)
    kw.pop("attention", None)
    return RefOps(**kw)

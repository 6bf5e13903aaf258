"""Reference implementations of every IR op in plain PyTorch (explicit forward AND backward, no autograd).

This backend is (a) the numerical oracle for the CUDA kernels, (b) the CPU path
used by the fp32 plumbing tests and by gloo multi-rank tests, and (c) on a GPU
the "library" baseline arm (torch matmul -> cuBLAS, torch SDPA).  The CUDA
backend subclasses it and overrides the hot ops with hand-written sm_100a
kernels.

Op implementations are methods named after the op kind; each takes
``(ctx, op, *inputs)`` and returns a tuple of outputs (one per declared output).
A backward op may return ``None`` for a ``grad::`` output it has already
accumulated in place through ``ctx.grad_sink``.

Parity: csrc/src/runtime/ops/*.cpp (per-op forward/backward dispatch).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn.functional as TF

IGNORE_INDEX = -100


@dataclass
class MoEPlan:
    """Routing plan shared by permute / grouped GEMM / un-permute (all tensors live on the device)."""
    sorted_src: torch.Tensor  # [N*K] int64: flat (token*K + k) index of each permuted row
    counts: torch.Tensor  # [E] int32 rows per (local) expert
    offsets: torch.Tensor  # [E+1] int32 exclusive scan
    num_tokens: int
    top_k: int
    num_experts: int
    x_shape: Tuple[int, ...] = ()  # shape of the un-permuted activation
    local: Optional["MoEPlan"] = None  # set on an EP plan: the sender-side permutation
    ep: Any = None  # EP bookkeeping (send/recv splits)


class RefOps:
    name = "ref"

    def __init__(self, lmhead_chunk_rows: int = 4096):
        self.lmhead_chunk_rows = lmhead_chunk_rows

    # ------------------------------------------------------------------ helpers
    def compute_dtype(self, t: torch.Tensor):
        return torch.float32 if t.dtype in (torch.bfloat16, torch.float16) else t.dtype

    def rope_cos_sin(self, position_ids: torch.Tensor, rotary_dim: int, theta: float, scaling=None, max_pos=None):
        from ..config.rope import rope_inv_freq

        inv, att = rope_inv_freq(rotary_dim, theta, scaling, max_pos, device=position_ids.device)
        ang = position_ids.to(torch.float32).unsqueeze(-1) * inv  # [B,T,half]
        return ang.cos() * att, ang.sin() * att

    def _rope_tables(self, ctx, a, pos):
        """cos / sin for this op: multi-axis (t, h, w) positions when the op has ``mrope_section`` and the batch has them."""
        p3 = ctx.extras.get("mrope_position_ids") if a.get("mrope_section") else None
        if p3 is None:
            return self.rope_cos_sin(pos, a["rotary_dim"], a["rope_theta"], a.get("rope_scaling"), a.get("max_pos"))
        from ..config.rope import rope_inv_freq

        inv, att = rope_inv_freq(a["rotary_dim"], a["rope_theta"], a.get("rope_scaling"), a.get("max_pos"), device=pos.device)
        ang3 = p3.to(torch.float32).unsqueeze(-1) * inv  # [3, B, T, half]
        ang = ang3[0].clone()
        for axis in (1, 2):
            idx = slice(axis, a["mrope_section"][axis] * 3, 3)
            ang[..., idx] = ang3[axis][..., idx]
        return ang.cos() * att, ang.sin() * att

    # ------------------------------------------------------------------ generic torch-function op
    @staticmethod
    def _fn_kwargs(op, ctx=None):
        kw = {k: v for k, v in op.attrs.items() if k not in ("fn", "n_out", "n_in", "side_inputs", "pass_layer", "shared_in", "shared_out")}
        for name in op.attrs.get("side_inputs", ()):  # per-batch tensors outside the graph (None when the batch has none)
            kw[name] = ctx.extras.get(name) if ctx is not None else None
        if op.attrs.get("pass_layer"):
            kw["layer"] = ctx.layer if ctx is not None else None
        return kw

    # ``shared_out`` = [[key, output index], ...]: the output is also left in ``ctx.shared[key]`` for ops of LATER layers that
    # name the key in ``shared_in`` (they get it as a keyword tensor).  Their backward runs first and accumulates the gradient
    # of the shared tensor in ``ctx.shared_grad[key]``; the producer's backward adds it to that output's incoming gradient.
    # This is how a value crosses layer boundaries without being part of the (x, residual) interface of a block:
    # keys / values reused by later layers, per-layer input embeddings computed once at the top.
    def torch_fn(self, ctx, op, *ins):
        from .torch_fns import TORCH_FNS

        kw = self._fn_kwargs(op, ctx)
        for key in op.attrs.get("shared_in", ()):
            kw[key] = ctx.shared[key]
        with torch.no_grad():
            out = TORCH_FNS[op.attrs["fn"]](*ins, **kw)
        outs = out if isinstance(out, tuple) else (out,)
        for key, idx in op.attrs.get("shared_out", ()):
            ctx.shared[key] = outs[idx]
        return outs

    def torch_fn_backward(self, ctx, op, *args):
        from .torch_fns import TORCH_FNS

        n_out = op.attrs["n_out"]
        d_outs, ins = list(args[:n_out]), list(args[n_out:])
        for key, idx in op.attrs.get("shared_out", ()):
            extra = ctx.shared_grad.pop(key, None)
            if extra is not None:
                d_outs[idx] = extra if d_outs[idx] is None else d_outs[idx] + extra.to(d_outs[idx].dtype)
        req = []
        for i, t in enumerate(ins):
            if torch.is_tensor(t) and t.is_floating_point():
                ins[i] = t.detach().requires_grad_(True)
                req.append(i)
        kw = self._fn_kwargs(op, ctx)
        shared = []
        for key in op.attrs.get("shared_in", ()):
            kw[key] = ctx.shared[key].detach().requires_grad_(True)
            shared.append(key)
        with torch.enable_grad():
            out = TORCH_FNS[op.attrs["fn"]](*ins, **kw)
            outs = out if isinstance(out, tuple) else (out,)
            pairs = [(o, d) for o, d in zip(outs, d_outs) if d is not None and torch.is_tensor(o) and o.requires_grad]
            gs = torch.autograd.grad([o for o, _ in pairs], [ins[i] for i in req] + [kw[k] for k in shared],
                                     [d.to(o.dtype) if torch.is_tensor(d) else torch.full_like(o, float(d)) for o, d in pairs], allow_unused=True)
        res = [None] * len(ins)
        for i, g in zip(req, gs):
            res[i] = g
        for key, g in zip(shared, gs[len(req):]):
            if g is not None:
                ctx.shared_grad[key] = g if key not in ctx.shared_grad else ctx.shared_grad[key] + g
        return tuple(res)

    # ------------------------------------------------------------------ simple ops
    def zeros(self, ctx, op):
        shape = ctx.eval_shape(op.attrs["shape"])
        return (torch.zeros(shape, dtype=ctx.dtype_of(op.attrs.get("dtype", "act")), device=ctx.device),)

    def add(self, ctx, op, a, b):
        return (a + b,)

    def mul(self, ctx, op, a, b):
        return (a * b,)

    def scale(self, ctx, op, a):
        return (a * op.attrs["factor"],)

    def view(self, ctx, op, a):
        return (a.reshape(ctx.eval_shape(op.attrs["shape"])),)

    def silu(self, ctx, op, x):
        return (TF.silu(x),)

    def silu_backward(self, ctx, op, dy, x):
        xf = x.float()
        s = torch.sigmoid(xf)
        return ((dy.float() * s * (1 + xf * (1 - s))).to(x.dtype),)

    def gelu(self, ctx, op, x):
        return (TF.gelu(x, approximate="tanh"),)

    def gelu_backward(self, ctx, op, dy, x):
        xf = x.float()
        c = math.sqrt(2.0 / math.pi)
        u = c * (xf + 0.044715 * xf ** 3)
        t = torch.tanh(u)
        d = 0.5 * (1 + t) + 0.5 * xf * (1 - t * t) * c * (1 + 3 * 0.044715 * xf * xf)
        return ((dy.float() * d).to(x.dtype),)

    # ------------------------------------------------------------------ embedding
    def embedding(self, ctx, op, token_ids, weight):
        return (weight[token_ids.long()].to(ctx.act_dtype),)

    def embedding_backward(self, ctx, op, d_x, token_ids):
        pname = op.outputs[0]
        C = d_x.shape[-1]
        tgt, acc = ctx.grad_target(pname)
        if tgt is None:
            return (None,)
        if not acc:
            tgt.zero_()
        tgt.index_add_(0, token_ids.reshape(-1).long(), d_x.reshape(-1, C).to(tgt.dtype))
        return (None,)

    # ------------------------------------------------------------------ norms
    def rmsnorm(self, ctx, op, x, w):
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1) + op.attrs["eps"])
        y = xf * rstd.unsqueeze(-1) * w.float()
        return y.to(x.dtype), rstd

    def fused_residual_rmsnorm(self, ctx, op, residual, x, w):
        r = residual + x
        y, rstd = self.rmsnorm(ctx, op, r, w)
        return r, y, rstd

    def rmsnorm_backward(self, ctx, op, dy, x, w, rstd, d_res):
        xf, dyf = x.float(), dy.float()
        xhat = xf * rstd.unsqueeze(-1)
        dn = dyf * w.float()
        dx = rstd.unsqueeze(-1) * (dn - xhat * (dn * xhat).mean(-1, keepdim=True))
        if d_res is not None:
            dx = dx + d_res.float()
        dw = (dyf * xhat).reshape(-1, x.shape[-1]).sum(0)
        return dx.to(x.dtype), dw

    # ------------------------------------------------------------------ matmul
    def matmul(self, ctx, op, x, w, bias):
        y = ctx.recipe.forward_matmul(ctx, op, x, w, bias) if ctx.recipe is not None else None
        if y is None:
            y = TF.linear(x, w.to(x.dtype), bias.to(x.dtype) if bias is not None else None)
        if ctx.lora is not None:
            y = ctx.lora.forward(ctx, op, x, y)
        return (y,)

    def matmul_backward(self, ctx, op, dy, x, w):
        K = x.shape[-1]
        N = dy.shape[-1]
        dy2, x2 = dy.reshape(-1, N), x.reshape(-1, K)
        r = ctx.recipe.backward_matmul(ctx, op, dy2, x2, w) if ctx.recipe is not None else None
        if r is not None:
            dx, dw = r
        else:
            dx = dy2 @ w.to(dy.dtype)
            dw = self._wgrad(ctx, op.outputs[1], dy2, x2)
        if ctx.lora is not None:
            extra = ctx.lora.backward(ctx, op, dy2, x2)
            if extra is not None:
                dx = dx + extra
        db = None
        if op.outputs[2] is not None:
            db = dy2.float().sum(0)
        return dx.reshape(x.shape), dw, db

    def _wgrad(self, ctx, pname, dy2, x2):
        """dW = dy^T x, accumulated straight into the gradient buffer when one is bound."""
        tgt, acc = ctx.grad_target(pname)
        if tgt is None:
            return None  # frozen parameter (e.g. LoRA base weight): no weight gradient
        if tgt.dtype == dy2.dtype and tgt.is_contiguous():
            if acc:
                tgt.addmm_(dy2.t(), x2)
            else:
                torch.mm(dy2.t(), x2, out=tgt)
        else:
            g = (dy2.t() @ x2).to(tgt.dtype)
            if acc:
                tgt.add_(g)
            else:
                tgt.copy_(g)
        return None

    # ------------------------------------------------------------------ qk-norm + rope
    def qkv_qk_norm_rope(self, ctx, op, qkv, qw, kw, pos):
        a = op.attrs
        Hq, Hkv, D, R = a["num_q_heads"], a["num_kv_heads"], a["head_dim"], a["rotary_dim"]
        lead = qkv.shape[:-1]
        x = qkv.float().reshape(*lead, Hq + 2 * Hkv, D)
        q, k, v = x[..., :Hq, :], x[..., Hq:Hq + Hkv, :], x[..., Hq + Hkv:, :]
        q_rstd = k_rstd = None
        if qw is not None:
            q_rstd = torch.rsqrt(q.pow(2).mean(-1) + a["eps"])
            k_rstd = torch.rsqrt(k.pow(2).mean(-1) + a["eps"])
            q = q * q_rstd.unsqueeze(-1) * qw.float()
            k = k * k_rstd.unsqueeze(-1) * kw.float()
        cos, sin = self._rope_tables(ctx, a, pos)
        q, k = self._rope(q, cos, sin, R, False), self._rope(k, cos, sin, R, False)
        out = torch.cat([q, k, v], dim=-2).reshape(qkv.shape).to(qkv.dtype)
        return out, q_rstd, k_rstd

    @staticmethod
    def _rope(x, cos, sin, R, conj):
        # x [..., H, D]; cos/sin [..., R/2] broadcast over heads
        h = R // 2
        c, s = cos.unsqueeze(-2), sin.unsqueeze(-2)
        if conj:
            s = -s
        x1, x2, rest = x[..., :h], x[..., h:R], x[..., R:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)

    def qkv_qk_norm_rope_backward(self, ctx, op, dy, qkv, qw, kw, q_rstd, k_rstd, pos):
        a = op.attrs
        Hq, Hkv, D, R = a["num_q_heads"], a["num_kv_heads"], a["head_dim"], a["rotary_dim"]
        lead = qkv.shape[:-1]
        g = dy.float().reshape(*lead, Hq + 2 * Hkv, D)
        x = qkv.float().reshape(*lead, Hq + 2 * Hkv, D)
        cos, sin = self._rope_tables(ctx, a, pos)
        gq, gk, gv = g[..., :Hq, :], g[..., Hq:Hq + Hkv, :], g[..., Hq + Hkv:, :]
        gq, gk = self._rope(gq, cos, sin, R, True), self._rope(gk, cos, sin, R, True)
        dqw = dkw = None
        if qw is not None:
            def nb(gy, xin, w, rstd):
                xhat = xin * rstd.unsqueeze(-1)
                dn = gy * w.float()
                dx = rstd.unsqueeze(-1) * (dn - xhat * (dn * xhat).mean(-1, keepdim=True))
                return dx, (gy * xhat).reshape(-1, D).sum(0)
            gq, dqw = nb(gq, x[..., :Hq, :], qw, q_rstd)
            gk, dkw = nb(gk, x[..., Hq:Hq + Hkv, :], kw, k_rstd)
        dx = torch.cat([gq, gk, gv], dim=-2).reshape(qkv.shape).to(qkv.dtype)
        return dx, dqw, dkw

    # ------------------------------------------------------------------ attention
    def _split_heads(self, qkv, a):
        Hq, Hkv, D = a["num_q_heads"], a["num_kv_heads"], a["head_dim"]
        B, T = qkv.shape[0], qkv.shape[1]
        x = qkv.reshape(B, T, Hq + 2 * Hkv, D)
        return x[:, :, :Hq], x[:, :, Hq:Hq + Hkv], x[:, :, Hq + Hkv:]

    # ------------------------------------------------------------------ attention against a key / value prefix (chunked sequences)
    @staticmethod
    def _prefix_mask(Tc, q0, k0, kn, a, device):
        """Additive mask for queries at absolute positions q0.. against keys k0..k0+kn."""
        qi = (q0 + torch.arange(Tc, device=device))[:, None]
        kj = (k0 + torch.arange(kn, device=device))[None, :]
        ok = kj <= qi if a.get("causal", True) else torch.ones(Tc, kn, dtype=torch.bool, device=device)
        if a.get("window", 0):
            ok = ok & ((qi - kj) < a["window"])
        return torch.zeros(Tc, kn, device=device).masked_fill(~ok, float("-inf"))

    def _chunk_attention(self, ctx, op, qkv):
        """Queries of the current chunk against all keys up to its end, one key block (= chunk) at a time with a running
        log-sum-exp, so the score matrix never exceeds chunk x chunk."""
        a, cs = op.attrs, ctx.chunk
        if ctx.doc_ids is not None:
            raise NotImplementedError("chunked-sequence training does not combine with packed documents")
        Hq, Hkv, D = a["num_q_heads"], a["num_kv_heads"], a["head_dim"]
        scale = a.get("softmax_scale") or 1.0 / math.sqrt(D)
        q, k, v = self._split_heads(qkv, a)
        B, Tc = qkv.shape[:2]
        cs.store_kv(ctx.layer, k, v)
        G, c, L = Hq // Hkv, cs.index, cs.chunk_len
        qf = q.float().permute(0, 2, 1, 3)
        m = torch.full((B, Hq, Tc), float("-inf"), device=qkv.device)
        den = torch.zeros(B, Hq, Tc, device=qkv.device)
        acc = torch.zeros(B, Hq, Tc, D, device=qkv.device)
        for j in range(c + 1):
            kn = Tc if j == c else L
            kf = cs.k[ctx.layer][:, j * L:j * L + kn].float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
            vf = cs.v[ctx.layer][:, j * L:j * L + kn].float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
            s = qf @ kf.transpose(-1, -2) * scale + self._prefix_mask(Tc, c * L, j * L, kn, a, qkv.device)
            m_new = torch.maximum(m, s.amax(-1))
            safe = torch.where(torch.isfinite(m_new), m_new, torch.zeros_like(m_new))  # rows with nothing visible yet
            alpha = torch.exp(torch.where(torch.isfinite(m), m - safe, torch.full_like(m, float("-inf"))))
            p = torch.exp(s - safe.unsqueeze(-1))
            den = den * alpha + p.sum(-1)
            acc = acc * alpha.unsqueeze(-1) + p @ vf
            m = m_new
        o = acc / den.unsqueeze(-1)
        lse = m + torch.log(den)
        return o.permute(0, 2, 1, 3).reshape(B, Tc, Hq * D).to(qkv.dtype), lse.permute(0, 2, 1).contiguous()

    def _chunk_attention_backward(self, ctx, op, d_att, qkv, att, lse):
        a, cs = op.attrs, ctx.chunk
        Hq, Hkv, D = a["num_q_heads"], a["num_kv_heads"], a["head_dim"]
        scale = a.get("softmax_scale") or 1.0 / math.sqrt(D)
        B, Tc = qkv.shape[:2]
        G, c, L = Hq // Hkv, cs.index, cs.chunk_len
        q, _, _ = self._split_heads(qkv, a)
        qf = q.float().permute(0, 2, 1, 3)
        do = d_att.float().reshape(B, Tc, Hq, D).permute(0, 2, 1, 3)
        o = att.float().reshape(B, Tc, Hq, D).permute(0, 2, 1, 3)
        delta = (do * o).sum(-1, keepdim=True)
        lse_h = lse.permute(0, 2, 1).unsqueeze(-1)
        dk_acc, dv_acc = cs.grad_buffers(ctx.layer)
        dq = torch.zeros_like(qf)
        for j in range(c + 1):
            kn = Tc if j == c else L
            rows = slice(j * L, j * L + kn)
            kf = cs.k[ctx.layer][:, rows].float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
            vf = cs.v[ctx.layer][:, rows].float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
            s = qf @ kf.transpose(-1, -2) * scale + self._prefix_mask(Tc, c * L, j * L, kn, a, qkv.device)
            p = torch.exp(s - lse_h)
            ds = p * (do @ vf.transpose(-1, -2) - delta) * scale
            dq += ds @ kf
            dk_acc[:, rows] += (ds.transpose(-1, -2) @ qf).reshape(B, Hkv, G, kn, D).sum(2).permute(0, 2, 1, 3)
            dv_acc[:, rows] += (p.transpose(-1, -2) @ do).reshape(B, Hkv, G, kn, D).sum(2).permute(0, 2, 1, 3)
        own = slice(c * L, c * L + Tc)  # by now these rows also hold what the later chunks contributed
        out = torch.cat([dq.permute(0, 2, 1, 3), dk_acc[:, own], dv_acc[:, own]], dim=2)
        return (out.reshape(qkv.shape).to(qkv.dtype),)

    def flash_attention(self, ctx, op, qkv):
        if ctx.chunk is not None:
            return self._chunk_attention(ctx, op, qkv)
        a = op.attrs
        Hq, Hkv, D = a["num_q_heads"], a["num_kv_heads"], a["head_dim"]
        scale = a.get("softmax_scale") or 1.0 / math.sqrt(D)
        q, k, v = self._split_heads(qkv, a)
        B, T = qkv.shape[:2]
        if qkv.is_cuda:
            return self._attention_library(ctx, op, q, k, v, scale)
        G = Hq // Hkv
        qf = q.float().permute(0, 2, 1, 3)  # B,Hq,T,D
        kf = k.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
        vf = v.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
        s = qf @ kf.transpose(-1, -2) * scale
        s = s + self._mask(T, a, s.device, ctx.doc_ids)
        lse = torch.logsumexp(s, dim=-1)  # B,Hq,T
        o = torch.exp(s - lse.unsqueeze(-1)) @ vf
        att = o.permute(0, 2, 1, 3).reshape(B, T, Hq * D).to(qkv.dtype)
        return att, lse.permute(0, 2, 1).contiguous()

    @staticmethod
    def _mask(T, a, device, doc_ids=None):
        i = torch.arange(T, device=device)
        ok = torch.ones(T, T, dtype=torch.bool, device=device)
        if a.get("causal", True):
            ok &= i[:, None] >= i[None, :]
        if a.get("window", 0):
            ok &= (i[:, None] - i[None, :]) < a["window"]
        m = torch.zeros(T, T, device=device).masked_fill(~ok, float("-inf"))
        if doc_ids is not None:  # packed documents: tokens attend within their own document only
            same = doc_ids[:, :, None] == doc_ids[:, None, :]
            m = m.unsqueeze(0).expand(doc_ids.shape[0], T, T).masked_fill(~same, float("-inf")).unsqueeze(1)
        return m

    def flash_attention_backward(self, ctx, op, d_att, qkv, att, lse):
        if ctx.chunk is not None:
            return self._chunk_attention_backward(ctx, op, d_att, qkv, att, lse)
        a = op.attrs
        Hq, Hkv, D = a["num_q_heads"], a["num_kv_heads"], a["head_dim"]
        scale = a.get("softmax_scale") or 1.0 / math.sqrt(D)
        B, T = qkv.shape[:2]
        if qkv.is_cuda:
            return self._attention_library_backward(ctx, op, d_att, qkv, att, lse)
        G = Hq // Hkv
        q, k, v = self._split_heads(qkv, a)
        qf = q.float().permute(0, 2, 1, 3)
        kf = k.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
        vf = v.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
        do = d_att.float().reshape(B, T, Hq, D).permute(0, 2, 1, 3)
        o = att.float().reshape(B, T, Hq, D).permute(0, 2, 1, 3)
        s = qf @ kf.transpose(-1, -2) * scale + self._mask(T, a, qkv.device, ctx.doc_ids)
        p = torch.exp(s - lse.permute(0, 2, 1).unsqueeze(-1))
        dv = p.transpose(-1, -2) @ do
        dp = do @ vf.transpose(-1, -2)
        delta = (do * o).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dq = ds @ kf
        dk = ds.transpose(-1, -2) @ qf
        dk = dk.reshape(B, Hkv, G, T, D).sum(2)
        dv = dv.reshape(B, Hkv, G, T, D).sum(2)
        out = torch.cat([dq.permute(0, 2, 1, 3), dk.permute(0, 2, 1, 3), dv.permute(0, 2, 1, 3)], dim=2)
        return (out.reshape(qkv.shape).to(qkv.dtype),)

    # library attention on a GPU: torch SDPA (cuDNN / flash kernels); the autograd node is kept as the "lse" slot
    def _attention_library(self, ctx, op, q, k, v, scale):
        a = op.attrs
        B, T = q.shape[:2]
        with torch.enable_grad():
            qh = q.transpose(1, 2).detach().requires_grad_(ctx.training)
            kh = k.transpose(1, 2).detach().requires_grad_(ctx.training)
            vh = v.transpose(1, 2).detach().requires_grad_(ctx.training)
            if ctx.doc_ids is not None or a.get("window", 0):
                # packed documents / sliding window: an explicit boolean mask (True = attend), never the plain causal shortcut
                allowed = self._mask(T, a, q.device, ctx.doc_ids) == 0
                allowed = allowed if allowed.dim() == 4 else allowed[None, None]
                o = TF.scaled_dot_product_attention(qh, kh, vh, attn_mask=allowed, scale=scale, enable_gqa=a["num_q_heads"] != a["num_kv_heads"])
            else:
                o = TF.scaled_dot_product_attention(qh, kh, vh, is_causal=a.get("causal", True), scale=scale,
                                                    enable_gqa=a["num_q_heads"] != a["num_kv_heads"])
        att = o.detach().transpose(1, 2).reshape(B, T, -1)
        return att, _AutogradHandle(o, (qh, kh, vh)) if ctx.training else None

    def _attention_library_backward(self, ctx, op, d_att, qkv, att, handle):
        a = op.attrs
        B, T = qkv.shape[:2]
        do = d_att.reshape(B, T, a["num_q_heads"], a["head_dim"]).transpose(1, 2)
        dq, dk, dv = torch.autograd.grad(handle.out, handle.inputs, do)
        out = torch.cat([dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)], dim=2)
        return (out.reshape(qkv.shape),)

    # ------------------------------------------------------------------ swiglu
    def swiglu(self, ctx, op, x):
        M = x.shape[-1] // 2
        up, gate = x[..., :M].float(), x[..., M:].float()
        return ((TF.silu(gate) * up).to(x.dtype),)

    # ------------------------------------------------------------------ tiled MLP (long context)
    def _mlp_tile_fwd(self, xc, up_w, down_w):
        u = TF.linear(xc, up_w.to(xc.dtype))
        a = self.swiglu(None, None, u)[0]
        return u, a, TF.linear(a, down_w.to(xc.dtype))

    def tiled_mlp(self, ctx, op, x, up_w, down_w):
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        rows = max(1, int(op.attrs["tile_rows"]))
        y = torch.empty(x2.shape[0], down_w.shape[0], dtype=x.dtype, device=x.device)
        for s in range(0, x2.shape[0], rows):
            y[s:s + rows] = self._mlp_tile_fwd(x2[s:s + rows], up_w, down_w)[2]
        return (y.reshape(*x.shape[:-1], down_w.shape[0]),)

    def tiled_mlp_backward(self, ctx, op, dy, x, up_w, down_w):
        C = x.shape[-1]
        x2, dy2 = x.reshape(-1, C), dy.reshape(-1, dy.shape[-1])
        rows = max(1, int(op.attrs["tile_rows"]))
        dx = torch.empty_like(x2)
        g_up, acc_up = ctx.grad_target(op.outputs[1])
        g_down, acc_down = ctx.grad_target(op.outputs[2])
        for s in range(0, x2.shape[0], rows):
            xc, dyc = x2[s:s + rows], dy2[s:s + rows]
            u, a, _ = self._mlp_tile_fwd(xc, up_w, down_w)          # recompute this tile
            da = dyc @ down_w.to(dyc.dtype)
            du = self.swiglu_backward(None, None, da, u)[0]
            dx[s:s + rows] = du @ up_w.to(du.dtype)
            for tgt, acc, lhs, rhs in ((g_down, acc_down, dyc, a), (g_up, acc_up, du, xc)):
                if tgt is not None:
                    g = (lhs.t().float() @ rhs.float()).to(tgt.dtype)
                    tgt.add_(g) if (acc or s > 0) else tgt.copy_(g)
        return dx.reshape(x.shape), None, None

    def swiglu_backward(self, ctx, op, dy, x):
        M = x.shape[-1] // 2
        up, gate = x[..., :M].float(), x[..., M:].float()
        s = torch.sigmoid(gate)
        g = dy.float()
        d_up = g * gate * s
        d_gate = g * up * s * (1 + gate * (1 - s))
        return (torch.cat([d_up, d_gate], dim=-1).to(x.dtype),)

    # ------------------------------------------------------------------ LM head + loss
    def _drop_ignored_rows(self, ctx, op, x, w, targets):
        """Optional compaction before the LM head: rows whose target is ignored (prompt tokens of an instruction dataset,
        padding) contribute neither loss nor gradient, so only the other rows go through the vocabulary GEMMs.  The row count
        is data dependent: one host sync per micro-batch sizes the compacted problem.  Returns None when nothing applies.
        Parity: lmhead_drop_ignored_rows (csrc/src/runtime/core/runtime_options.h)."""
        if not getattr(ctx.ex.options, "lmhead_drop_ignored_rows", False) or getattr(ctx, "_dropping", False):
            return None
        if ctx.row_weights is not None or ctx.kd is not None or ctx.want_token_losses:
            return None
        if not torch.is_tensor(x):  # a quantised activation wrapper (plain tensors also have a ``dequantize`` method: do not ask for it)
            x = x.hp if getattr(x, "hp", None) is not None else x.dequantize()
        C = x.shape[-1]
        x2, t = x.reshape(-1, C), targets.reshape(-1)
        keep = (t != IGNORE_INDEX).nonzero(as_tuple=False).squeeze(1)
        if keep.numel() == t.numel():
            return None
        pad = (-keep.numel()) % 8 if keep.numel() else 8  # keep the row count a multiple of 8 (GEMM tile alignment); padded rows are ignored ones
        if pad:
            ignored = (t == IGNORE_INDEX).nonzero(as_tuple=False).squeeze(1)[:pad]
            keep = torch.cat([keep, ignored])
        ctx._dropping = True
        try:
            out = self.fused_lm_head_loss(ctx, op, x2.index_select(0, keep).unsqueeze(0), w, t.index_select(0, keep).unsqueeze(0))
        finally:
            ctx._dropping = False
        if ctx.training:
            dx = torch.zeros_like(x2)
            dx.index_copy_(0, keep, ctx.stash[op.outputs[0]].reshape(-1, C))
            ctx.stash[op.outputs[0]] = dx.reshape(x.shape)
        return out

    def fused_lm_head_loss(self, ctx, op, x, w, targets):
        """Returns the summed CE over valid tokens.  In training mode also computes d_x (stashed) and d_w now.
        Objective hooks (see ExecContext): per-token weights on the log-likelihood gradient, top-K distillation."""
        dropped = self._drop_ignored_rows(ctx, op, x, w, targets)
        if dropped is not None:
            return dropped
        C = x.shape[-1]
        x2, t = x.reshape(-1, C), targets.reshape(-1).long()
        n = x2.shape[0]
        loss = torch.zeros((), dtype=torch.float32, device=x.device)
        train = ctx.training
        dx = torch.empty_like(x2) if train else None
        pname = None
        if train:
            pname = "grad::" + op.inputs[1]
            tgt, acc = ctx.grad_target(pname)
        scale = ctx.loss_scale
        cap = op.attrs.get("softcap", 0.0)
        rows = self.lmhead_chunk_rows
        rw = ctx.row_weights.reshape(-1).float() if getattr(ctx, "row_weights", None) is not None else None
        kd = getattr(ctx, "kd", None)
        ce_w = float(kd.get("ce_weight", 1.0)) if kd else 1.0
        kd_w = float(kd["weight"]) if kd else 0.0
        kd_idx = kd["idx"].reshape(n, -1).long() if kd else None
        kd_logp = kd["logp"].reshape(n, -1).float() if kd else None
        tok_all = torch.zeros(n, dtype=torch.float32, device=x.device) if getattr(ctx, "want_token_losses", False) else None
        kd_all = torch.zeros(n, dtype=torch.float32, device=x.device) if (kd and tok_all is not None) else None
        kd_total = torch.zeros((), dtype=torch.float32, device=x.device)
        for s in range(0, n, rows):
            xs, ts = x2[s:s + rows], t[s:s + rows]
            logits = (xs @ w.to(xs.dtype).t()).float()
            if cap:
                th = torch.tanh(logits / cap)
                logits = th * cap
            valid = ts != IGNORE_INDEX
            tsafe = ts.clamp_min(0)
            lse = torch.logsumexp(logits, dim=-1)
            tok_loss = (lse - logits.gather(1, tsafe[:, None]).squeeze(1)) * valid
            loss += tok_loss.sum()
            if tok_all is not None:
                tok_all[s:s + rows] = tok_loss
            if kd:
                ki, kl = kd_idx[s:s + rows], kd_logp[s:s + rows]
                pk = torch.exp(kl)
                kd_tok = (pk * (kl - (logits.gather(1, ki) - lse[:, None]))).sum(1) * valid
                kd_total += kd_tok.sum()
                if kd_all is not None:
                    kd_all[s:s + rows] = kd_tok
            if train:
                q = torch.exp(logits - lse[:, None])
                w_row = torch.ones_like(lse) if rw is None else rw[s:s + rows]
                w_row = w_row * ce_w
                p = q * w_row[:, None]
                p.scatter_add_(1, tsafe[:, None], -w_row[:, None])
                if kd:
                    p += kd_w * pk.sum(1, keepdim=True) * q
                    p.scatter_add_(1, ki, -kd_w * pk)
                p *= (valid[:, None] * scale)
                if cap:
                    p *= (1 - th * th)
                pd = p.to(xs.dtype)
                dx[s:s + rows] = pd @ w.to(xs.dtype)
                if tgt is not None:
                    g = pd.t() @ xs
                    if acc:
                        tgt.add_(g.to(tgt.dtype))
                    else:
                        tgt.copy_(g.to(tgt.dtype))
                        acc = True
        if train:
            ctx.stash[op.outputs[0]] = dx.reshape(x.shape)
        if tok_all is not None:
            ctx.stash["token_losses"] = tok_all
            if kd_all is not None:
                ctx.stash["token_kd"] = kd_all
        if kd:
            loss = ce_w * loss + kd_w * kd_total
        return (loss,)

    def fused_lm_head_loss_backward(self, ctx, op, d_loss, x, w, targets, loss):
        dx = ctx.stash.pop(op.inputs[4])
        return dx, None

    # ------------------------------------------------------------------ MoE
    def moe_router(self, ctx, op, x, rw):
        a = op.attrs
        E, K = a["num_experts"], a["top_k"]
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        logits = x2.float() @ rw.float().t()
        probs = torch.softmax(logits, -1) if a["scoring"] == "softmax" else torch.sigmoid(logits)
        tw, ti = torch.topk(probs, K, dim=-1)
        if a["norm_topk_prob"]:
            tw = tw / tw.sum(-1, keepdim=True)
        N = x2.shape[0]
        counts = torch.bincount(ti.reshape(-1), minlength=E).float()
        aux = a["aux_loss_coef"] * E * ((counts / N) * probs.mean(0)).sum()
        if a.get("z_loss_coef", 0.0):
            aux = aux + a["z_loss_coef"] * torch.logsumexp(logits, -1).pow(2).mean()
        ctx.record_moe_stats(counts, probs)
        lead = x.shape[:-1]
        return tw.reshape(*lead, K), ti.to(torch.int32).reshape(*lead, K), aux

    def moe_router_backward(self, ctx, op, d_tw, d_aux, x, rw, tw, ti):
        a = op.attrs
        E, K = a["num_experts"], a["top_k"]
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        N = x2.shape[0]
        logits = x2.float() @ rw.float().t()
        soft = a["scoring"] == "softmax"
        probs = torch.softmax(logits, -1) if soft else torch.sigmoid(logits)
        til = ti.reshape(N, K).long()
        sel = probs.gather(1, til)
        d_sel = torch.zeros_like(sel)
        if d_tw is not None:
            g = d_tw.reshape(N, K).float()
            if a["norm_topk_prob"]:
                ssum = sel.sum(-1, keepdim=True)
                d_sel = g / ssum - (g * sel).sum(-1, keepdim=True) / (ssum * ssum)
            else:
                d_sel = g
        d_probs = torch.zeros_like(probs).scatter_add_(1, til, d_sel)
        d_logits_extra = None
        if d_aux is not None:
            da = d_aux if torch.is_tensor(d_aux) else torch.tensor(float(d_aux), device=x.device)
            counts = torch.bincount(til.reshape(-1), minlength=E).float()
            d_probs = d_probs + da * a["aux_loss_coef"] * E * (counts / N) / N
            if a.get("z_loss_coef", 0.0):
                lse = torch.logsumexp(logits, -1, keepdim=True)
                d_logits_extra = da * a["z_loss_coef"] * 2 * lse / N * torch.softmax(logits, -1)
        if soft:
            d_logits = probs * (d_probs - (d_probs * probs).sum(-1, keepdim=True))
        else:
            d_logits = d_probs * probs * (1 - probs)
        if d_logits_extra is not None:
            d_logits = d_logits + d_logits_extra
        dx = (d_logits @ rw.float()).to(x.dtype).reshape(x.shape)
        drw = d_logits.t() @ x2.float()
        return dx, drw

    def moe_permute(self, ctx, op, x, ti):
        a = op.attrs
        E, K = a["num_experts"], a["top_k"]
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        flat = ti.reshape(-1).long()
        sorted_src = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=E).to(torch.int32)
        offsets = torch.zeros(E + 1, dtype=torch.int32, device=x.device)
        offsets[1:] = torch.cumsum(counts, 0)
        xp = x2[sorted_src // K]
        return xp, MoEPlan(sorted_src, counts, offsets, x2.shape[0], K, E, tuple(x.shape))

    def moe_permute_backward(self, ctx, op, d_xp, plan):
        plan = plan.local or plan
        C = d_xp.shape[-1]
        dx = torch.zeros(plan.num_tokens, C, dtype=torch.float32, device=d_xp.device)
        dx.index_add_(0, plan.sorted_src // plan.top_k, d_xp.float())
        return (dx.to(d_xp.dtype).reshape(plan.x_shape),)

    def _expert_ranges(self, plan):
        off = plan.offsets.tolist()  # host sync: reference path only
        return [(e, off[e], off[e + 1]) for e in range(len(off) - 1) if off[e + 1] > off[e]]

    def moe_grouped_gemm(self, ctx, op, x, w, plan):
        y = torch.empty(x.shape[0], w.shape[1], dtype=x.dtype, device=x.device)
        w = ctx.local_experts(w)
        if getattr(plan, "send_idx", None) is not None:     # least-loaded step: foreign expert slots, their weights shipped by the owners
            w = ctx.ep.extend_weights(ctx, op.attrs.get("role", ""), w, plan)
        for e, s, t in self._expert_ranges(plan):
            y[s:t] = x[s:t] @ w[e].to(x.dtype).t()
        if ctx.lora is not None:
            y = ctx.lora.forward_grouped(ctx, op, x, y, plan)
        return (y,)

    def moe_grouped_gemm_backward(self, ctx, op, dy, x, w, plan):
        dx = torch.empty_like(x)
        wl = ctx.local_experts(w)
        tgt, acc = ctx.grad_target(op.outputs[1])
        if tgt is not None:
            tgt = ctx.local_experts(tgt)
            if not acc:
                tgt.zero_()
        spilled = getattr(plan, "send_idx", None) is not None
        if spilled:
            role = op.attrs.get("role", "")
            n_native = wl.shape[0]
            wl = ctx.ep.extend_weights(ctx, role, wl, plan)
            d_foreign = [torch.zeros(wl.shape[1:], dtype=torch.float32, device=x.device) for _ in range(wl.shape[0] - n_native)]
        for e, s, t in self._expert_ranges(plan):
            dx[s:t] = dy[s:t] @ wl[e].to(dy.dtype)
            if tgt is not None:
                if spilled and e >= n_native:
                    d_foreign[e - n_native] += (dy[s:t].t() @ x[s:t]).float()
                else:
                    tgt[e] += (dy[s:t].t() @ x[s:t]).to(tgt.dtype)
        if spilled and tgt is not None:   # the helpers' share of every expert's weight gradient returns to the expert's owner
            for e_local, gsum in ctx.ep.return_weight_grads(ctx, role, d_foreign, plan, torch.zeros((1,) + tuple(wl.shape[1:]), dtype=torch.float32, device=x.device)):
                tgt[e_local] += gsum.to(tgt.dtype)
        if ctx.lora is not None:
            extra = ctx.lora.backward_grouped(ctx, op, dy, x, plan)
            if extra is not None:
                dx = dx + extra
        return dx, None

    @staticmethod
    def _row_experts(plan, rows: int, device):
        """(expert of each permuted row, whether the row is a real routed row) from the plan's device-side offsets / counts:
        no host sync, and padding rows between experts (kernel plans pad each expert's range) are marked invalid.
        Plans with a ``counts`` tensor keep [E + 1] range starts in ``offsets``; expert-parallel receive plans keep
        [El + 1 starts, overflow, El real counts] in one tensor."""
        # an expert-parallel receive plan describes the rows as they lie on the experts' owner; its ``local`` is the sender's plan
        p = plan if hasattr(plan, "recv_splits") else (getattr(plan, "local", None) or plan)
        layout = getattr(p, "layout", None)     # kernel expert-parallel plans: the full [El + 1 starts, overflow, El real counts] tensor
        off = (layout if (layout is not None and getattr(p, "counts", None) is None) else p.offsets).to(device=device, dtype=torch.int64)
        counts = getattr(p, "counts", None)
        if counts is not None:
            E = counts.numel()
            counts = counts.to(device=device, dtype=torch.int64)
        else:
            E = (off.numel() - 2) // 2
            counts = off[E + 2:2 * E + 2]
        r = torch.arange(rows, device=device)
        eid = torch.bucketize(r, off[1:E + 1].contiguous(), right=True).clamp_max(E - 1)
        valid = (r - off[eid]) < counts[eid]
        return eid, valid

    def moe_expert_bias_add(self, ctx, op, y, bias, plan):
        eid, valid = self._row_experts(plan, y.shape[0], y.device)
        b = ctx.local_experts(bias)
        if getattr(plan, "send_idx", None) is not None:     # least-loaded step: the foreign slots' biases come from their owners
            b = ctx.ep.extend_weights(ctx, "bias:" + str(op.outputs[0]), b, plan)
        return (y + (b.to(y.dtype)[eid] * valid.unsqueeze(-1)),)

    def moe_expert_bias_add_backward(self, ctx, op, dy, bias, plan):
        eid, valid = self._row_experts(plan, dy.shape[0], dy.device)
        tgt, acc = ctx.grad_target(op.outputs[1])
        if tgt is not None:
            tgt = ctx.local_experts(tgt)
            spilled = getattr(plan, "send_idx", None) is not None
            slots = int(plan.counts.numel()) if spilled else tgt.shape[0]
            g = torch.zeros((slots,) + tuple(tgt.shape[1:]), dtype=torch.float32, device=dy.device).index_add_(0, eid, dy.float() * valid.unsqueeze(-1))
            if spilled:     # the foreign slots' bias gradients return to the experts' owners
                n = tgt.shape[0]
                back = ctx.ep.return_weight_grads(ctx, "bias", [g[i] for i in range(n, slots)], plan, g[:1])
                g = g[:n].clone()
                for e_local, part in back:
                    g[e_local] += part
            if acc:
                tgt.add_(g.to(tgt.dtype))
            else:
                tgt.copy_(g.to(tgt.dtype))
        return dy, None

    def moe_unpermute(self, ctx, op, yp, tw, plan):
        plan = plan.local or plan
        N, K = plan.num_tokens, plan.top_k
        C = yp.shape[-1]
        wflat = tw.reshape(-1).float()[plan.sorted_src]  # weight of each permuted row
        y = torch.zeros(N, C, dtype=torch.float32, device=yp.device)
        y.index_add_(0, plan.sorted_src // K, yp.float() * wflat[:, None])
        return (y.to(yp.dtype).reshape(plan.x_shape),)

    def moe_unpermute_backward(self, ctx, op, dy, yp, tw, plan):
        plan = plan.local or plan
        N, K = plan.num_tokens, plan.top_k
        C = yp.shape[-1]
        dy2 = dy.reshape(N, C).float()
        tok = plan.sorted_src // K
        wflat = tw.reshape(-1).float()[plan.sorted_src]
        d_yp = (dy2[tok] * wflat[:, None]).to(yp.dtype)
        d_w_sorted = (yp.float() * dy2[tok]).sum(-1)
        d_tw = torch.zeros(N * K, dtype=torch.float32, device=yp.device)
        d_tw[plan.sorted_src] = d_w_sorted
        return d_yp, d_tw.reshape(tw.shape)

    # EP ops: identity unless a parallel context overrides them
    def ep_dispatch(self, ctx, op, xp, plan):
        return ctx.ep.dispatch(ctx, xp, plan) if ctx.ep is not None else (xp, plan)

    def ep_combine(self, ctx, op, y, plan):
        return (ctx.ep.combine(ctx, y, plan),) if ctx.ep is not None else (y,)

    def ep_dispatch_backward(self, ctx, op, dy, plan):
        return (ctx.ep.dispatch_backward(ctx, dy, plan),) if ctx.ep is not None else (dy,)


class _AutogradHandle:
    """Keeps a library attention call's autograd graph alive between forward and backward."""

    def __init__(self, out, inputs):
        self.out, self.inputs = out, inputs

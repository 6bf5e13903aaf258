"""Functional op emitters used inside ``nn.Module.forward``.

Each function records one IR op on the active tracer and returns proxies for its
outputs.  The op vocabulary is the fused-op granularity the runtime executes
(one op ≈ one kernel or one GEMM), matching the reference's op registry
(csrc/src/runtime/executor/op_registrations.cpp; typed signatures in
surogate/dsl/primitives/*.py).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

from .ir import Shape, dim_mul
from .nn import Proxy, current_tracer


def _t():
    return current_tracer()


def zeros(shape: Shape, dtype: str = "act", name: str = "zeros") -> Proxy:
    return _t().emit("zeros", [], [(name, tuple(shape), dtype)], shape=list(shape), dtype=dtype)[0]


def embedding(token_ids: Proxy, weight: Proxy, name: str = "x0") -> Proxy:
    C = weight.shape[1]
    return _t().emit("embedding", [token_ids, weight], [(name, token_ids.shape + (C,), "act")])[0]


def add(a: Proxy, b: Proxy, name: str = "add") -> Proxy:
    return _t().emit("add", [a, b], [(name, a.shape, a.dtype)])[0]


def mul(a: Proxy, b: Proxy, name: str = "mul") -> Proxy:
    return _t().emit("mul", [a, b], [(name, a.shape, a.dtype)])[0]


def scale(a: Proxy, s: float, name: str = "scale") -> Proxy:
    return _t().emit("scale", [a], [(name, a.shape, a.dtype)], factor=float(s))[0]


def view(a: Proxy, shape: Shape, name: str = "view") -> Proxy:
    return _t().emit("view", [a], [(name, tuple(shape), a.dtype)], shape=list(shape))[0]


def rmsnorm(x: Proxy, weight: Proxy, eps: float, name: str = "ln") -> Tuple[Proxy, Proxy]:
    y, rstd = _t().emit("rmsnorm", [x, weight], [(name, x.shape, "act"), (f"{name}_rstd", x.shape[:-1], "fp32")], eps=eps)
    return y, rstd


def fused_residual_rmsnorm(residual: Proxy, x: Proxy, weight: Proxy, eps: float, name: str = "ln",
                           res_name: str = "res") -> Tuple[Proxy, Proxy, Proxy]:
    """residual_out = residual + x ; y = rmsnorm(residual_out) * weight.  Returns (residual_out, y, rstd)."""
    r, y, rstd = _t().emit(
        "fused_residual_rmsnorm", [residual, x, weight],
        [(res_name, x.shape, "act"), (name, x.shape, "act"), (f"{name}_rstd", x.shape[:-1], "fp32")], eps=eps)
    return r, y, rstd


def matmul(x: Proxy, w: Proxy, bias: Optional[Proxy] = None, name: str = "mm", role: str = "") -> Proxy:
    """y[..., N] = x[..., K] @ w[N, K]^T (+ bias).  ``role`` tags the GEMM for recipes/LoRA (qkv, out, mlp_up, ...)."""
    N, K = w.shape
    assert x.shape[-1] == K, f"[E011] matmul shape mismatch: {x.shape} @ {w.shape}^T"
    return _t().emit("matmul", [x, w, bias], [(name, x.shape[:-1] + (N,), "act")], transpose="NT", role=role)[0]


def qkv_qk_norm_rope(qkv: Proxy, q_norm_w: Optional[Proxy], k_norm_w: Optional[Proxy], position_ids: Proxy, *,
                     num_q_heads: int, num_kv_heads: int, head_dim: int, eps: float, rope_theta: float,
                     rotary_dim: Optional[int] = None, rope_scaling=None, max_pos: Optional[int] = None, mrope_section=None,
                     name: str = "qkv_rope") -> Tuple[Proxy, Optional[Proxy], Optional[Proxy]]:
    """Per-head RMSNorm on Q and K (optional) followed by rotary embedding on the packed [.., (Hq+2Hkv)*D] tensor.
    ``mrope_section`` = (t, h, w): when the batch carries the side input ``mrope_position_ids`` [3, B, T], frequency i uses the
    height positions if i % 3 == 1 and i < 3h, the width positions if i % 3 == 2 and i < 3w, else the temporal ones."""
    use_norm = q_norm_w is not None
    lead = qkv.shape[:-1]
    outs = _t().emit(
        "qkv_qk_norm_rope", [qkv, q_norm_w, k_norm_w, position_ids],
        [(name, qkv.shape, "act"),
         ("q_rstd", lead + (num_q_heads,), "fp32") if use_norm else None,
         ("k_rstd", lead + (num_kv_heads,), "fp32") if use_norm else None],
        num_q_heads=num_q_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, eps=eps, rope_theta=rope_theta,
        rotary_dim=rotary_dim or head_dim, **({"rope_scaling": dict(rope_scaling), "max_pos": max_pos} if rope_scaling else {}),
        **({"mrope_section": [int(v) for v in mrope_section]} if mrope_section else {}))
    return outs[0], outs[1], outs[2]


def flash_attention(qkv: Proxy, *, num_q_heads: int, num_kv_heads: int, head_dim: int, causal: bool = True,
                    window: int = 0, softmax_scale: Optional[float] = None, name: str = "att") -> Tuple[Proxy, Proxy]:
    lead = qkv.shape[:-1]
    att, lse = _t().emit(
        "flash_attention", [qkv], [(name, lead + (num_q_heads * head_dim,), "act"), ("lse", lead + (num_q_heads,), "fp32")],
        num_q_heads=num_q_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, causal=causal, window=window,
        softmax_scale=softmax_scale)
    return att, lse


def swiglu(x: Proxy, name: str = "swiglu") -> Proxy:
    """x = [up | gate] on the last dim (up first); y = silu(gate) * up."""
    M2 = x.shape[-1]
    return _t().emit("swiglu", [x], [(name, x.shape[:-1] + (M2 // 2,), "act")])[0]


def tiled_mlp(x: Proxy, up_w: Proxy, down_w: Proxy, tile_rows: int, name: str = "mlp_down") -> Proxy:
    """Gated MLP evaluated over row tiles: y = down(swiglu(up(x))) without ever holding the [tokens, 2*d_ff] intermediate for more
    than ``tile_rows`` tokens; the backward recomputes each tile.  For very long sequences, where that intermediate dominates
    activation memory."""
    return _t().emit("tiled_mlp", [x, up_w, down_w], [(name, x.shape[:-1] + (down_w.shape[0],), "act")], tile_rows=int(tile_rows))[0]


def silu(x: Proxy, name: str = "silu") -> Proxy:
    return _t().emit("silu", [x], [(name, x.shape, x.dtype)])[0]


def gelu(x: Proxy, name: str = "gelu") -> Proxy:
    return _t().emit("gelu", [x], [(name, x.shape, x.dtype)])[0]


def fused_lm_head_loss(x: Proxy, w: Proxy, targets: Proxy, name: str = "loss", softcap: float = 0.0) -> Proxy:
    """Sum over valid (target != -100) tokens of cross-entropy(x @ w^T, target); logits never fully materialised."""
    return _t().emit("fused_lm_head_loss", [x, w, targets], [(name, (), "fp32")], softcap=softcap)[0]


# ---------------------------------------------------------------------------- MoE

def moe_router(x: Proxy, router_w: Proxy, *, top_k: int, norm_topk_prob: bool, aux_loss_coef: float,
               z_loss_coef: float = 0.0, scoring: str = "softmax") -> Tuple[Proxy, Proxy, Proxy]:
    """Router GEMM (fp32 logits) -> softmax/sigmoid -> top-k (+ optional renormalise) -> aux/z losses.

    Returns (topk_weights [N,K] fp32, topk_index [N,K] int32, aux_loss scalar)."""
    lead = x.shape[:-1]
    E = router_w.shape[0]
    w, idx, aux = _t().emit(
        "moe_router", [x, router_w],
        [("topk_weights", lead + (top_k,), "fp32"), ("topk_index", lead + (top_k,), "int32"), ("moe_aux_loss", (), "fp32")],
        num_experts=E, top_k=top_k, norm_topk_prob=norm_topk_prob, aux_loss_coef=aux_loss_coef,
        z_loss_coef=z_loss_coef, scoring=scoring)
    return w, idx, aux


def moe_permute(x: Proxy, topk_index: Proxy, *, num_experts: int, top_k: int) -> Tuple[Proxy, Proxy]:
    """Sort token copies by expert.  Returns (permuted rows [N*K, C], routing plan (opaque))."""
    C = x.shape[-1]
    n = 1
    for d in x.shape[:-1]:
        n = dim_mul(n, d)
    xp, plan = _t().emit("moe_permute", [x, topk_index], [("moe_permuted", (dim_mul(n, top_k), C), "act"), ("moe_plan", (), "opaque")],
                         num_experts=num_experts, top_k=top_k)
    return xp, plan


def ep_dispatch(xp: Proxy, plan: Proxy) -> Tuple[Proxy, Proxy]:
    """Expert-parallel all-to-all: rows travel to the rank owning their expert.  Identity when ep_size == 1."""
    y, plan2 = _t().emit("ep_dispatch", [xp, plan], [("ep_recv", xp.shape, "act"), ("ep_plan", (), "opaque")])
    return y, plan2


def ep_combine(y: Proxy, plan: Proxy) -> Proxy:
    return _t().emit("ep_combine", [y, plan], [("ep_back", y.shape, "act")])[0]


def moe_grouped_gemm(x: Proxy, w: Proxy, plan: Proxy, name: str, role: str) -> Proxy:
    """Per-expert GEMM: rows of ``x`` are grouped by expert according to ``plan``; w is [E, N, K]."""
    E, N, K = w.shape
    return _t().emit("moe_grouped_gemm", [x, w, plan], [(name, (x.shape[0], N), "act")], role=role)[0]


def moe_expert_bias_add(y: Proxy, bias: Proxy, plan: Proxy, name: str = "moe_biased") -> Proxy:
    """Adds each expert's bias row ([E, N]) to the permuted rows that belong to that expert."""
    return _t().emit("moe_expert_bias_add", [y, bias, plan], [(name, y.shape, "act")])[0]


def moe_unpermute(y: Proxy, topk_weights: Proxy, plan: Proxy, out_shape: Shape, name: str = "moe_out") -> Proxy:
    """Weighted sum of each token's K expert outputs, back in token order."""
    return _t().emit("moe_unpermute", [y, topk_weights, plan], [(name, tuple(out_shape), "act")])[0]


# ---------------------------------------------------------------------------- generic torch-function op

def torch_fn(fn: str, inputs: Sequence[Optional[Proxy]], out_specs: Sequence[Tuple[str, Shape, str]], **attrs):
    """An op implemented by a registered PyTorch function (``runtime/torch_fns.py``); its backward is obtained by replaying the
    function under autograd.  This is how architectures outside the tuned kernel set (sliding-window / sink attention,
    state-space mixers, short convolutions, biased MoE ...) run through the same graph machinery."""
    outs = _t().emit("torch_fn", list(inputs), list(out_specs), fn=fn, n_out=len(out_specs), **attrs)
    return outs[0] if len(outs) == 1 else tuple(outs)

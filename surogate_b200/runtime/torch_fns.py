"""PyTorch implementations behind the generic ``torch_fn`` op.

Architectures outside the hand-tuned set (sliding-window and sink attention, GeGLU / ReLU^2 MLPs, LayerNorm, biased
clamp-SwiGLU experts, short convolutions, state-space and delta-rule mixers) are expressed with these functions; the
executor calls them in forward and replays them under autograd for backward.  Each function takes tensors first and
plain-Python keyword attributes after, and returns a tensor or a tuple of tensors.

Parity: csrc/src/runtime/ops/ (gelu_glu, relu2, layernorm, gpt_oss_moe_act, moe_expert_bias_add, mamba_*,
chunk_gated_delta_rule), csrc/src/runtime/attention/attention_custom.cu (sliding window / sinks).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Optional

import torch
import torch.nn.functional as F

TORCH_FNS: Dict[str, Callable] = {}


def register(name: str):
    def deco(fn):
        TORCH_FNS[name] = fn
        return fn

    return deco


# ---------------------------------------------------------------------------------------------- element-wise / norms
@register("geglu")
def geglu(x, *, approximate: str = "tanh", gate_first: bool = False):
    """x = [up | gate] (or [gate | up]); y = gelu(gate) * up."""
    a, b = x.chunk(2, dim=-1)
    up, gate = (b, a) if gate_first else (a, b)
    if x.is_cuda and approximate == "tanh":      # one run-time compiled kernel each way instead of five element-wise passes
        from ..ops.jit import GEGLU_TANH

        return GEGLU_TANH(gate.contiguous(), up.contiguous())
    return F.gelu(gate.float(), approximate=approximate).to(x.dtype) * up


@register("relu2")
def relu2(x):
    if x.is_cuda:
        from ..ops.jit import RELU2

        return RELU2(x)
    return F.relu(x).square()


@register("layernorm")
def layernorm(x, w, b, *, eps: float = 1e-5):
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float() if b is not None else None, eps).to(x.dtype)


@register("rmsnorm_offset")
def rmsnorm_offset(x, w, *, eps: float = 1e-6, offset: float = 1.0):
    """Gemma-style RMSNorm: y = x / rms(x) * (offset + w), computed in fp32."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (offset + w.float())).to(x.dtype)


@register("sigmoid_gate_mul")
def sigmoid_gate_mul(x, w, y):
    """y * sigmoid(x @ w^T) with a [1, C] weight: the per-token gate on a shared expert."""
    return y * torch.sigmoid(F.linear(x.float(), w.float())).to(y.dtype)


@register("visual_scatter")
def visual_scatter(x, *, visual_pos_masks=None, visual_embeds=None):
    """Token embeddings with the rows at image / video placeholder positions replaced by the vision tower's outputs
    (``visual_embeds`` [n_visual, C] in row-major order of the mask).  No gradient reaches the replaced embedding rows."""
    if visual_pos_masks is None or visual_embeds is None:
        return x + 0
    m = visual_pos_masks.to(torch.bool)
    return torch.where(m.unsqueeze(-1), torch.zeros_like(x), x).masked_scatter(m.unsqueeze(-1), visual_embeds.to(x.dtype))


@register("deepstack_add")
def deepstack_add(y, *, layer=None, visual_pos_masks=None, deepstack_visual_embeds=None):
    """Add the ``layer``-th intermediate vision feature to the hidden state at the visual positions (first few layers only)."""
    if visual_pos_masks is None or not deepstack_visual_embeds or layer is None or layer >= len(deepstack_visual_embeds):
        return y + 0
    m = visual_pos_masks.to(torch.bool).unsqueeze(-1)
    return y + torch.zeros_like(y).masked_scatter(m, deepstack_visual_embeds[layer].to(y.dtype))


@register("softplus_gate_mul")
def softplus_gate_mul(att, gate, *, head_dim: int):
    """att [.., H*D] scaled by softplus(gate): one gate per head ([.., H]) or per channel ([.., H*D])."""
    g = F.softplus(gate.float())
    if g.shape[-1] != att.shape[-1]:
        g = g.repeat_interleave(head_dim, dim=-1)
    return (att.float() * g).to(att.dtype)


@register("sigmoid_bias_router")
def sigmoid_bias_router(x, router_w, bias, *, top_k: int, scaling_factor: float = 1.0):
    """Sigmoid router with a selection-only bias: experts are chosen by sigmoid(logits) + bias, weighted by the unbiased
    scores renormalised over the chosen ones, times ``scaling_factor``.  Returns (weights fp32 [.., K], indices int32 [.., K])."""
    lead = x.shape[:-1]
    scores = torch.sigmoid(F.linear(x.reshape(-1, x.shape[-1]).float(), router_w.float()))
    idx = torch.topk(scores.detach() + bias.float(), top_k, dim=-1).indices
    w = scores.gather(1, idx)
    w = w / w.sum(-1, keepdim=True) * scaling_factor
    return w.reshape(*lead, top_k), idx.to(torch.int32).reshape(*lead, top_k)


@register("scale_by_buffer")
def scale_by_buffer(x, s):
    """x times a checkpoint buffer (a value that is loaded and saved but never trained)."""
    return x * s.detach().to(x.dtype)


@register("gemma4_qkv_norm_rope")
def gemma4_qkv_norm_rope(qkv, qn_w, kn_w, pos, *, num_q_heads: int, num_kv_heads: int, head_dim: int, eps: float, rope_theta: float, rope_scaling=None,
                         k_eq_v: bool = False):
    """Packed [.., (Hq + 2 Hkv) D] (or [.., (Hq + Hkv) D] when values reuse the key projection) -> packed q, k, v with
    RMSNorm(scale) on q and k, scale-free RMSNorm on v, and rotary embedding over the whole head (pairs i, i + D/2)."""
    from ..config.rope import rope_inv_freq

    lead = qkv.shape[:-1]
    Hq, Hkv, D = num_q_heads, num_kv_heads, head_dim
    x = qkv.float().reshape(*lead, -1, D)
    q, k = x[..., :Hq, :], x[..., Hq:Hq + Hkv, :]
    v = k if k_eq_v else x[..., Hq + Hkv:, :]
    q, k, v = _rms(q, eps) * qn_w.float(), _rms(k, eps) * kn_w.float(), _rms(v, eps)
    inv, att = rope_inv_freq(D, rope_theta, rope_scaling, None, device=qkv.device)
    ang = pos.float().unsqueeze(-1) * inv
    cos, sin = (ang.cos() * att).unsqueeze(-2), (ang.sin() * att).unsqueeze(-2)

    def rope(t):
        a, b = t[..., :D // 2], t[..., D // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)

    return torch.cat([rope(q), rope(k), v], dim=-2).reshape(*lead, (Hq + 2 * Hkv) * D).to(qkv.dtype)


@register("gemma4_q_norm_rope_shared")
def gemma4_q_norm_rope_shared(q, qn_w, pos, *, num_q_heads: int, num_kv_heads: int, head_dim: int, eps: float, rope_theta: float, rope_scaling=None, **shared):
    """Query side of a layer that reuses an earlier layer's keys and values: normalise and rotate q, take k and v from the
    producer's packed tensor (the one keyword tensor in ``shared``)."""
    from ..config.rope import rope_inv_freq

    (kv,) = shared.values()
    lead, Hq, Hkv, D = q.shape[:-1], num_q_heads, num_kv_heads, head_dim
    qh = _rms(q.float().reshape(*lead, Hq, D), eps) * qn_w.float()
    inv, att = rope_inv_freq(D, rope_theta, rope_scaling, None, device=q.device)
    ang = pos.float().unsqueeze(-1) * inv
    cos, sin = (ang.cos() * att).unsqueeze(-2), (ang.sin() * att).unsqueeze(-2)
    a, b = qh[..., :D // 2], qh[..., D // 2:]
    qh = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    return torch.cat([qh.reshape(*lead, Hq * D).to(q.dtype), kv[..., Hq * D:].to(q.dtype)], dim=-1)


@register("slice_last")
def slice_last(x, *, start: int, size: int):
    return x[..., start:start + size].contiguous()


@register("keep_params")
def keep_params(x, *params):
    """Identity on ``x``.  Lists parameters that exist in the checkpoint but are not used by this layer (so they are loaded,
    kept and exported unchanged)."""
    return x + 0


@register("gemma4_pli")
def gemma4_pli(x, token_ids, emb_w, proj_w, norm_w, *, n_layers: int, d_pli: int, eps: float):
    """Per-layer input embeddings: a second (scaled) token embedding of width L * P plus a projection of the main embedding,
    RMS-normalised per layer, averaged with 1/sqrt(2).  Returns (x unchanged, per-layer inputs [B, T, L, P])."""
    B, T, C = x.shape
    emb = F.embedding(token_ids.long(), emb_w).float() * float(torch.tensor(d_pli ** 0.5).to(emb_w.dtype))
    proj = F.linear(x.float(), proj_w.float()) * (C ** -0.5)
    proj = _rms(proj.reshape(B, T, n_layers, d_pli), eps) * norm_w.float()
    return x + 0, ((proj + emb.reshape(B, T, n_layers, d_pli)) * (2.0 ** -0.5)).to(x.dtype)


@register("gemma4_pli_apply")
def gemma4_pli_apply(h, gate_w, proj_w, norm_w, *, layer: int, pli, eps: float):
    """gelu(h W_gate) * per-layer input of this layer -> projection back to the model width -> RMSNorm."""
    g = F.gelu(F.linear(h, gate_w).float(), approximate="tanh") * pli[:, :, layer].float()
    return (_rms(F.linear(g.to(h.dtype), proj_w).float(), eps) * norm_w.float()).to(h.dtype)


@register("gemma4_router")
def gemma4_router(x, proj_w, scale, per_expert_scale, *, top_k: int, eps: float):
    """Scale-free RMSNorm, a learned per-channel scale and 1/sqrt(C), linear -> softmax -> top-k renormalised to sum 1, then a
    learned per-expert multiplier.  Returns (weights fp32 [.., K], indices int32 [.., K])."""
    lead, C = x.shape[:-1], x.shape[-1]
    h = _rms(x.reshape(-1, C).float(), eps) * scale.float() * (C ** -0.5)
    probs = torch.softmax(F.linear(h, proj_w.float()), dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    w = w / w.sum(-1, keepdim=True) * per_expert_scale.float()[idx]
    return w.reshape(*lead, top_k), idx.to(torch.int32).reshape(*lead, top_k)


@register("scale_by")
def scale_by(x, s):
    return x * s.to(x.dtype)


@register("softcap")
def softcap(x, *, cap: float):
    if x.is_cuda:
        from ..ops.jit import SOFTCAP

        return SOFTCAP(x, cap=float(cap))
    return torch.tanh(x.float() / cap).mul(cap).to(x.dtype)


# ---------------------------------------------------------------------------------------------- attention
@register("attention_general")
def attention_general(qkv, sinks=None, *, num_q_heads: int, num_kv_heads: int, head_dim: int, window: int = 0, softmax_scale: Optional[float] = None,
                      softcap: float = 0.0, causal: bool = True, v_head_dim: Optional[int] = None):
    """Grouped-query attention on packed [B, T, (Hq + 2 Hkv) D] with optional sliding window, logit soft-capping and learned
    per-head sink logits (a virtual key that only absorbs probability mass)."""
    B, T = qkv.shape[:2]
    Hq, Hkv, D = num_q_heads, num_kv_heads, head_dim
    x = qkv.reshape(B, T, Hq + 2 * Hkv, D)
    q, k, v = x[:, :, :Hq], x[:, :, Hq:Hq + Hkv], x[:, :, Hq + Hkv:]
    G = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    s = qf @ kf.transpose(-1, -2) * (softmax_scale or 1.0 / math.sqrt(D))
    if softcap:
        s = torch.tanh(s / softcap) * softcap
    i = torch.arange(T, device=qkv.device)
    ok = torch.ones(T, T, dtype=torch.bool, device=qkv.device)
    if causal:
        ok &= i[:, None] >= i[None, :]
    if window:
        ok &= (i[:, None] - i[None, :]) < window
    s = s.masked_fill(~ok, float("-inf"))
    if sinks is not None:
        sk = sinks.float().reshape(1, Hq, 1, 1).expand(B, Hq, T, 1)
        p = torch.softmax(torch.cat([s, sk], dim=-1), dim=-1)[..., :-1]
    else:
        p = torch.softmax(s, dim=-1)
    o = p @ vf
    return o.permute(0, 2, 1, 3).reshape(B, T, Hq * D).to(qkv.dtype)


# ---------------------------------------------------------------------------------------------- GPT-OSS style MoE
@register("topk_softmax_router")
def topk_softmax_router(x, router_w, router_b, *, top_k: int):
    """linear (+ bias) -> top-k logits -> softmax over the chosen k.  Returns (weights fp32 [.., K], indices int32 [.., K])."""
    lead = x.shape[:-1]
    logits = F.linear(x.reshape(-1, x.shape[-1]).float(), router_w.float(), router_b.float() if router_b is not None else None)
    top_v, top_i = torch.topk(logits, top_k, dim=-1)
    return torch.softmax(top_v, dim=-1).reshape(*lead, top_k), top_i.to(torch.int32).reshape(*lead, top_k)


@register("clamped_glu_interleaved")
def clamped_glu_interleaved(h, *, alpha: float = 1.702, limit: float = 7.0):
    """[.., 2M] with gate and up interleaved (even columns gate, odd columns up): gate clamped above, up clamped on both sides at
    ``limit``, y = (up + 1) * gate * sigmoid(alpha * gate)."""
    hf = h.float()
    gate, up = hf[..., ::2].clamp(max=limit), hf[..., 1::2].clamp(min=-limit, max=limit)
    return ((up + 1) * gate * torch.sigmoid(gate * alpha)).to(h.dtype)


@register("moe_biased_clamp_swiglu")
def moe_biased_clamp_swiglu(x, router_w, router_b, gate_up, gate_up_b, down, down_b, *, top_k: int, alpha: float = 1.702, limit: float = 7.0):
    """Router = linear(+bias) -> top-k -> softmax over the k selected logits.  Experts: interleaved (gate, up) columns with
    biases, gate clamped above and up clamped on both sides at ``limit``, y = (up + 1) * gate * sigmoid(alpha * gate), then the
    biased down projection.  gate_up [E, C, 2M], down [E, M, C] (input-major, as stored in the checkpoint)."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    logits = F.linear(x2.float(), router_w.float(), router_b.float())
    top_v, top_i = torch.topk(logits, top_k, dim=-1)
    w = torch.softmax(top_v, dim=-1)
    out = torch.zeros_like(x2, dtype=torch.float32)
    E = router_w.shape[0]
    for e in range(E):
        tok, slot = torch.where(top_i == e)
        if tok.numel() == 0:
            continue
        h = x2[tok].float() @ gate_up[e].float() + gate_up_b[e].float()
        gate, up = h[..., ::2].clamp(max=limit), h[..., 1::2].clamp(min=-limit, max=limit)
        act = (up + 1) * gate * torch.sigmoid(gate * alpha)
        y = act @ down[e].float() + down_b[e].float()
        out.index_add_(0, tok, y * w[tok, slot, None])
    return out.reshape(shape).to(x.dtype)


# ---------------------------------------------------------------------------------------------- short convolution (LFM2)
@register("short_conv")
def short_conv(x, in_w, conv_w, out_w, in_b=None, conv_b=None, out_b=None, *, kernel: int = 3):
    """Gated depth-wise causal convolution: (B, C, x') = in_proj(x) split in three; y = out_proj(C * conv1d(B * x'))."""
    from ..ops.conv1d import causal_conv1d

    Bx, T, D = x.shape
    b, c, xx = F.linear(x, in_w, in_b).chunk(3, dim=-1)          # channels-last throughout: no transposes around the convolution
    conv = causal_conv1d((b * xx).contiguous(), conv_w.reshape(D, kernel), conv_b)
    return F.linear(c * conv, out_w, out_b)


# ---------------------------------------------------------------------------------------------- Mamba-2 mixer (Nemotron-H)
def _segsum(x):
    T = x.shape[-1]
    x = x[..., None].expand(*x.shape, T)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool, device=x.device), diagonal=-1)
    x = x.masked_fill(~mask, 0)
    seg = torch.cumsum(x, dim=-2)
    mask2 = torch.tril(torch.ones(T, T, dtype=torch.bool, device=x.device), diagonal=0)
    return seg.masked_fill(~mask2, float("-inf"))


def ssd_scan(xh, dt, A, Bm, Cm, D, *, chunk: int):
    """Structured state-space duality scan.  xh [B,T,H,P], dt [B,T,H] (after softplus), A [H] (negative), Bm/Cm [B,T,G,N], D [H]."""
    Bsz, T, H, P = xh.shape
    G, N = Bm.shape[2], Bm.shape[3]
    pad = (-T) % chunk
    if pad:
        xh, dt, Bm, Cm = (torch.cat([t, t.new_zeros(t.shape[0], pad, *t.shape[2:])], 1) for t in (xh, dt, Bm, Cm))
    Tp = T + pad
    rep = H // G
    Bh, Ch = Bm.repeat_interleave(rep, dim=2), Cm.repeat_interleave(rep, dim=2)
    xd = xh * dt[..., None]
    a = A[None, None, :] * dt  # [B,T,H]
    nc = Tp // chunk
    r = lambda t: t.reshape(Bsz, nc, chunk, *t.shape[2:])  # noqa: E731
    xd, a, Bh, Ch = r(xd), r(a), r(Bh), r(Ch)
    a = a.permute(0, 3, 1, 2)  # [B,H,c,l]
    a_cum = torch.cumsum(a, dim=-1)
    L = torch.exp(_segsum(a))
    y_diag = torch.einsum("bclhn,bcshn,bhcls,bcshp->bclhp", Ch, Bh, L, xd)
    decay_states = torch.exp(a_cum[..., -1:] - a_cum)
    states = torch.einsum("bclhn,bhcl,bclhp->bchpn", Bh, decay_states, xd)
    init = states.new_zeros(Bsz, 1, H, P, N)
    states = torch.cat([init, states], dim=1)
    decay_chunk = torch.exp(_segsum(F.pad(a_cum[..., -1], (1, 0))))
    new_states = torch.einsum("bhzc,bchpn->bzhpn", decay_chunk, states)
    states = new_states[:, :-1]
    y_off = torch.einsum("bclhn,bchpn,bhcl->bclhp", Ch, states, torch.exp(a_cum))
    y = (y_diag + y_off).reshape(Bsz, Tp, H, P)[:, :T]
    return y + xh[:, :T] * D[None, None, :, None]


@register("mamba2_mixer")
def mamba2_mixer(x, in_w, conv_w, conv_b, dt_bias, A_log, D, norm_w, out_w, *, num_heads: int, head_dim: int, n_groups: int, state_size: int,
                 conv_kernel: int = 4, chunk: int = 64, eps: float = 1e-5, in_b=None, out_b=None):
    """Mamba-2 block: in_proj -> (gate z, conv input [x, B, C], dt) -> causal depth-wise conv + SiLU -> SSD scan -> gated grouped
    RMSNorm -> out_proj."""
    Bsz, T, _ = x.shape
    H, P, G, N = num_heads, head_dim, n_groups, state_size
    inner = H * P
    proj = F.linear(x, in_w, in_b).float()
    z, xBC, dt = torch.split(proj, [inner, inner + 2 * G * N, H], dim=-1)
    from ..ops.conv1d import causal_conv1d

    xBC = causal_conv1d(xBC.contiguous(), conv_w.float().reshape(-1, conv_kernel), conv_b.float(), activation="silu")
    xs, Bm, Cm = torch.split(xBC, [inner, G * N, G * N], dim=-1)
    dt = F.softplus(dt + dt_bias.float())
    y = ssd_scan(xs.reshape(Bsz, T, H, P), dt, -torch.exp(A_log.float()), Bm.reshape(Bsz, T, G, N), Cm.reshape(Bsz, T, G, N), D.float(), chunk=chunk)
    y = y.reshape(Bsz, T, inner) * F.silu(z)
    yg = y.reshape(Bsz, T, G, inner // G)
    yg = yg * torch.rsqrt(yg.pow(2).mean(-1, keepdim=True) + eps)
    y = yg.reshape(Bsz, T, inner) * norm_w.float()
    return F.linear(y.to(x.dtype), out_w, out_b)


# ---------------------------------------------------------------------------------------------- gated delta rule (Qwen3.5 / Qwen3-Next)
def gated_delta_rule(q, k, v, g, beta, *, scale: Optional[float] = None, chunk: int = 64):
    """Gated delta rule  S_t = exp(g_t) S_{t-1} + beta_t k_t (v_t - exp(g_t) S_{t-1}^T k_t)^T,  o_t = S_t^T q_t,  evaluated chunk
    by chunk: inside a chunk of ``chunk`` positions the rank-one updates are folded into two triangular matrix products (the
    inverse of I + strict_lower(beta k k^T * decay) built by forward substitution), so the sequential part runs over T / chunk
    state updates made of matrix products instead of T outer products.  Short sequences use the step-by-step form.
    q, k [B,T,H,Dk]; v [B,T,H,Dv]; g [B,T,H] (log decay, <= 0); beta [B,T,H].
    Parity: surogate/kernels/triton/gated_delta_rule.py (chunk_gated_delta_rule)."""
    B, T, H, Dk = q.shape
    if T <= chunk:
        return gated_delta_rule_recurrent(q, k, v, g, beta, scale=scale)
    Dv = v.shape[-1]
    C = chunk
    q = F.normalize(q.float(), dim=-1) * (scale if scale is not None else Dk ** -0.5)
    k = F.normalize(k.float(), dim=-1)
    v, g, beta = v.float(), g.float(), beta.float()
    pad = (-T) % C
    if pad:  # padded steps: beta = 0 (no write), g = 0 (no decay), outputs dropped
        q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
        g, beta = F.pad(g, (0, 0, 0, pad)), F.pad(beta, (0, 0, 0, pad))
    N = (T + pad) // C
    # [B, H, N, C, D]
    q, k, v = (t.permute(0, 2, 1, 3).reshape(B, H, N, C, -1) for t in (q, k, v))
    g, beta = (t.permute(0, 2, 1).reshape(B, H, N, C) for t in (g, beta))
    gc = g.cumsum(-1)
    decay = torch.exp(gc.unsqueeze(-1) - gc.unsqueeze(-2)).tril()          # exp(gc_i - gc_j), i >= j
    kb, vb = k * beta.unsqueeze(-1), v * beta.unsqueeze(-1)
    strict = torch.ones(C, C, dtype=torch.bool, device=q.device).tril(-1)
    A = -(kb @ k.transpose(-1, -2) * decay).masked_fill(~strict, 0.0)
    rows = [A[..., 0, :]]
    for i in range(1, C):  # forward substitution: row i of (I - A_strict)^-1 - I from the rows above it
        prev = torch.stack(rows, dim=-2)                                   # [.., i, C]
        rows.append(A[..., i, :] + (A[..., i, :i].unsqueeze(-2) @ prev).squeeze(-2))
    Tm = torch.stack(rows, dim=-2) + torch.eye(C, device=q.device)
    w = Tm @ (kb * torch.exp(gc).unsqueeze(-1))
    u = Tm @ vb
    local = (q @ k.transpose(-1, -2) * decay).masked_fill(~(strict | torch.eye(C, dtype=torch.bool, device=q.device)), 0.0)
    q_in = q * torch.exp(gc).unsqueeze(-1)
    last = gc[..., -1]
    k_out = k * torch.exp(last.unsqueeze(-1) - gc).unsqueeze(-1)
    S = q.new_zeros(B, H, Dk, Dv)
    outs = []
    for n in range(N):
        v_new = u[:, :, n] - w[:, :, n] @ S
        outs.append(q_in[:, :, n] @ S + local[:, :, n] @ v_new)
        S = S * torch.exp(last[:, :, n])[..., None, None] + k_out[:, :, n].transpose(-1, -2) @ v_new
    o = torch.stack(outs, dim=2).reshape(B, H, N * C, Dv)[:, :, :T]
    return o.permute(0, 2, 1, 3)


def gated_delta_rule_recurrent(q, k, v, g, beta, *, scale: Optional[float] = None):
    """Recurrent form of the gated delta rule.  q,k [B,T,H,Dk], v [B,T,H,Dv], g [B,T,H] (log decay, <= 0), beta [B,T,H].
    S_t = exp(g_t) S_{t-1} + beta_t k_t (v_t - exp(g_t) S_{t-1}^T k_t)^T ; o_t = S_t^T q_t."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    q = F.normalize(q.float(), dim=-1) * (scale if scale is not None else Dk ** -0.5)
    k = F.normalize(k.float(), dim=-1)
    v, g, beta = v.float(), g.float(), beta.float()
    S = q.new_zeros(B, H, Dk, Dv)
    outs = []
    for t in range(T):
        S = S * torch.exp(g[:, t])[..., None, None]
        kv = torch.einsum("bhk,bhkv->bhv", k[:, t], S)
        delta = (v[:, t] - kv) * beta[:, t][..., None]
        S = S + torch.einsum("bhk,bhv->bhkv", k[:, t], delta)
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, t], S))
    return torch.stack(outs, dim=1)


@register("gated_delta_rule")
def gated_delta_rule_op(q, k, v, g, beta, *, scale: Optional[float] = None):
    return gated_delta_rule(q, k, v, g, beta, scale=scale).to(v.dtype)


# ---------------------------------------------------------------------------------------------- Nemotron-H style MoE
@register("sigmoid_group_router")
def sigmoid_group_router(x, gate_w, score_bias, *, top_k: int, n_group: int = 1, topk_group: int = 1, norm_topk_prob: bool = True,
                         routed_scaling_factor: float = 1.0):
    """Sigmoid router with a selection-only score bias and group-limited top-k (experts are chosen only inside the ``topk_group``
    best of ``n_group`` groups, a group's score being the sum of its two best experts).  Weights are the unbiased scores of the
    chosen experts, renormalised and scaled.  Returns (weights fp32 [.., K], indices int32 [.., K])."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    E = gate_w.shape[0]
    scores = torch.sigmoid(F.linear(x2.float(), gate_w.float()))
    choice = scores.detach() + score_bias.float()
    if n_group > 1:
        gs = choice.view(-1, n_group, E // n_group).topk(2, dim=-1)[0].sum(-1)
        gi = torch.topk(gs, k=topk_group, dim=-1, sorted=False)[1]
        gmask = torch.zeros_like(gs).scatter_(1, gi, 1.0)
        mask = gmask.unsqueeze(-1).expand(-1, n_group, E // n_group).reshape(-1, E).bool()
        choice = choice.masked_fill(~mask, 0.0)
    top_i = torch.topk(choice, k=top_k, dim=-1, sorted=False)[1]
    w = scores.gather(1, top_i)
    if norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    w = w * routed_scaling_factor
    return w.reshape(*lead, top_k), top_i.to(torch.int32).reshape(*lead, top_k)


@register("moe_sigmoid_relu2")
def moe_sigmoid_relu2(x, gate_w, score_bias, up, down, shared_up, shared_down, *, top_k: int, n_group: int = 1, topk_group: int = 1,
                      norm_topk_prob: bool = True, routed_scaling_factor: float = 1.0):
    """Sigmoid router with a selection-only score bias and group-limited top-k; non-gated ReLU^2 experts (up [E, M, C],
    down [E, C, M]) plus an always-on shared ReLU^2 expert."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    E = gate_w.shape[0]
    scores = torch.sigmoid(F.linear(x2.float(), gate_w.float()))
    choice = scores + score_bias.float()
    if n_group > 1:
        gs = choice.view(-1, n_group, E // n_group).topk(2, dim=-1)[0].sum(-1)
        gi = torch.topk(gs, k=topk_group, dim=-1, sorted=False)[1]
        gmask = torch.zeros_like(gs).scatter_(1, gi, 1.0)
        mask = gmask.unsqueeze(-1).expand(-1, n_group, E // n_group).reshape(-1, E).bool()
        choice = choice.masked_fill(~mask, 0.0)
    top_i = torch.topk(choice.detach(), k=top_k, dim=-1, sorted=False)[1]
    w = scores.gather(1, top_i)
    if norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    w = w * routed_scaling_factor
    out = torch.zeros_like(x2, dtype=torch.float32)
    for e in range(E):
        tok, slot = torch.where(top_i == e)
        if tok.numel() == 0:
            continue
        h = F.relu(F.linear(x2[tok].float(), up[e].float())).square()
        out.index_add_(0, tok, F.linear(h, down[e].float()) * w[tok, slot, None])
    shared = F.linear(F.relu(F.linear(x2.float(), shared_up.float())).square(), shared_down.float())
    return (out + shared).reshape(shape).to(x.dtype)


# ---------------------------------------------------------------------------------------------- Qwen3.5 / Qwen3-Next mixers
def _rms(x, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


@register("qwen35_gated_attention")
def qwen35_gated_attention(x, q_w, k_w, v_w, o_w, qn_w, kn_w, pos, *, num_q_heads: int, num_kv_heads: int, head_dim: int, eps: float, rope_theta: float,
                           rotary_dim: int):
    """Attention whose query projection also yields a per-channel output gate: q_proj -> [q | gate] per head, zero-centred
    QK RMSNorm, partial rotary embedding, causal GQA, output multiplied by sigmoid(gate) before o_proj."""
    B, T, _ = x.shape
    Hq, Hkv, D = num_q_heads, num_kv_heads, head_dim
    qg = F.linear(x, q_w).float().view(B, T, Hq, 2 * D)
    q, gate = qg[..., :D], qg[..., D:].reshape(B, T, Hq * D)
    k = F.linear(x, k_w).float().view(B, T, Hkv, D)
    v = F.linear(x, v_w).float().view(B, T, Hkv, D)
    q = _rms(q, eps) * (1.0 + qn_w.float())
    k = _rms(k, eps) * (1.0 + kn_w.float())
    half = rotary_dim // 2
    inv = rope_theta ** (-torch.arange(0, half, device=x.device, dtype=torch.float32) * 2.0 / rotary_dim)
    ang = pos.float().unsqueeze(-1) * inv
    cos, sin = ang.cos().unsqueeze(2), ang.sin().unsqueeze(2)

    def rope(t):
        a, b, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], dim=-1)

    q, k = rope(q), rope(k)
    G = Hq // Hkv
    qf = q.permute(0, 2, 1, 3)
    kf = k.permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    vf = v.permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    s = qf @ kf.transpose(-1, -2) * (D ** -0.5)
    i = torch.arange(T, device=x.device)
    s = s.masked_fill(~(i[:, None] >= i[None, :]), float("-inf"))
    o = (torch.softmax(s, dim=-1) @ vf).permute(0, 2, 1, 3).reshape(B, T, Hq * D)
    return F.linear((o * torch.sigmoid(gate)).to(x.dtype), o_w)


@register("qwen35_gated_delta_net")
def qwen35_gated_delta_net(x, qkv_w, z_w, b_w, a_w, conv_w, dt_bias, A_log, norm_w, out_w, *, num_k_heads: int, num_v_heads: int, head_k_dim: int,
                           head_v_dim: int, conv_kernel: int, eps: float):
    """Gated DeltaNet mixer: qkv projection -> causal depth-wise conv + SiLU -> L2-normalised q, k; per-head decay
    g = -exp(A_log) softplus(a + dt_bias) and write strength beta = sigmoid(b); gated delta rule; RMSNorm gated by silu(z)."""
    B, T, _ = x.shape
    Hk, Hv, Dk, Dv = num_k_heads, num_v_heads, head_k_dim, head_v_dim
    key_dim, value_dim = Hk * Dk, Hv * Dv
    from ..ops.conv1d import causal_conv1d

    mixed = causal_conv1d(F.linear(x, qkv_w).float().contiguous(), conv_w.float().reshape(-1, conv_kernel), None, activation="silu")
    q, k, v = torch.split(mixed, [key_dim, key_dim, value_dim], dim=-1)
    q, k, v = q.reshape(B, T, Hk, Dk), k.reshape(B, T, Hk, Dk), v.reshape(B, T, Hv, Dv)
    beta = torch.sigmoid(F.linear(x, b_w).float())
    g = -torch.exp(A_log.float()) * F.softplus(F.linear(x, a_w).float() + dt_bias.float())
    if Hv // Hk > 1:
        q, k = q.repeat_interleave(Hv // Hk, dim=2), k.repeat_interleave(Hv // Hk, dim=2)
    l2 = lambda t: t * torch.rsqrt((t * t).sum(-1, keepdim=True) + 1e-6)  # noqa: E731
    q, k = l2(q) * (Dk ** -0.5), l2(k)
    S = q.new_zeros(B, Hv, Dk, Dv)
    outs = []
    for t in range(T):
        S = S * torch.exp(g[:, t])[..., None, None]
        kv = torch.einsum("bhk,bhkv->bhv", k[:, t], S)
        S = S + torch.einsum("bhk,bhv->bhkv", k[:, t], (v[:, t] - kv) * beta[:, t][..., None])
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, t], S))
    o = torch.stack(outs, dim=1).reshape(-1, Dv)
    z = F.linear(x, z_w).float().reshape(-1, Dv)
    o = (norm_w.float() * _rms(o, eps)) * F.silu(z)
    return F.linear(o.reshape(B, T, value_dim).to(x.dtype), out_w)

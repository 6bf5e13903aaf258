"""Independent plain-PyTorch (autograd) implementations of the model families, used as oracles."""
import math

import torch
import torch.nn.functional as F


def rope(x, pos, theta):
    # x [B,T,H,D]
    D = x.shape[-1]
    inv = theta ** (-torch.arange(0, D // 2, dtype=torch.float32, device=x.device) * 2.0 / D)
    ang = pos.float()[..., None] * inv
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, :, None], torch.cat([ang.sin(), ang.sin()], -1)[:, :, None]
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return x * cos + torch.cat([-x2, x1], -1) * sin


def rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def attention(h, p, L, cfg, pos):
    B, T, C = h.shape
    Hq, Hkv, D = cfg["Hq"], cfg["Hkv"], cfg["D"]
    qkv = h @ p[f"blocks.{L}.qkv_weight"].t()
    if f"blocks.{L}.qkv_bias" in p:
        qkv = qkv + p[f"blocks.{L}.qkv_bias"]
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], -1)
    q, k, v = q.view(B, T, Hq, D), k.view(B, T, Hkv, D), v.view(B, T, Hkv, D)
    if cfg.get("qk_norm", True):
        q = rms(q, p[f"blocks.{L}.q_norm_weight"], cfg["eps"])
        k = rms(k, p[f"blocks.{L}.k_norm_weight"], cfg["eps"])
    q, k = rope(q, pos, cfg["theta"]), rope(k, pos, cfg["theta"])
    G = Hq // Hkv
    k, v = k.repeat_interleave(G, 2), v.repeat_interleave(G, 2)
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
    return o.transpose(1, 2).reshape(B, T, Hq * D) @ p[f"blocks.{L}.out_weight"].t()


def dense_mlp(h, p, L):
    u = h @ p[f"blocks.{L}.mlp_up_weight"].t()
    M = u.shape[-1] // 2
    return (F.silu(u[..., M:]) * u[..., :M]) @ p[f"blocks.{L}.mlp_down_weight"].t()


def moe_mlp(h, p, L, cfg):
    B, T, C = h.shape
    E, K = cfg["E"], cfg["K"]
    x = h.reshape(-1, C)
    logits = x @ p[f"blocks.{L}.router_weight"].t()
    probs = torch.softmax(logits.float(), -1)
    tw, ti = torch.topk(probs, K, -1)
    if cfg.get("norm_topk", True):
        tw = tw / tw.sum(-1, keepdim=True)
    y = torch.zeros_like(x)
    for e in range(E):
        tok, slot = (ti == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        u = x[tok] @ p[f"blocks.{L}.experts_gate_up"][e].t()
        M = u.shape[-1] // 2
        o = (F.silu(u[:, M:]) * u[:, :M]) @ p[f"blocks.{L}.experts_down"][e].t()
        y = y.index_add(0, tok, o * tw[tok, slot][:, None])
    N = x.shape[0]
    counts = torch.bincount(ti.reshape(-1), minlength=E).float()
    aux = cfg["aux_coef"] * E * ((counts / N) * probs.mean(0)).sum()
    return y.view(B, T, C), aux


def model_logits(p, tokens, cfg, pos=None):
    """Logits [B, T, V] of a dense model (same math as model_loss, in the dtype of the parameters)."""
    if pos is None:
        pos = torch.arange(tokens.shape[1], dtype=torch.int32)[None].expand(tokens.shape[0], -1)
    x = p["embedding"][tokens]
    for L in range(cfg["n_layers"]):
        h = rms(x, p[f"blocks.{L}.ln1_weight"], cfg["eps"])
        x = x + attention(h, p, L, cfg, pos)
        h = rms(x, p[f"blocks.{L}.ln2_weight"], cfg["eps"])
        x = x + dense_mlp(h, p, L)
    x = rms(x, p["final_norm"], cfg["eps"])
    w = p["lm_head"] if "lm_head" in p else p["embedding"]
    return x @ w.t()


def model_loss(p, tokens, pos, targets, cfg):
    """Returns (sum CE over valid tokens, sum of aux losses)."""
    x = p["embedding"][tokens]
    aux_total = torch.zeros((), dtype=torch.float32)
    for L in range(cfg["n_layers"]):
        h = rms(x, p[f"blocks.{L}.ln1_weight"], cfg["eps"])
        x = x + attention(h, p, L, cfg, pos)
        h = rms(x, p[f"blocks.{L}.ln2_weight"], cfg["eps"])
        if cfg.get("E"):
            y, aux = moe_mlp(h, p, L, cfg)
            aux_total = aux_total + aux
            x = x + y
        else:
            x = x + dense_mlp(h, p, L)
    x = rms(x, p["final_norm"], cfg["eps"])
    w = p["lm_head"] if "lm_head" in p else p["embedding"]
    logits = x @ w.t()
    loss = F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), targets.reshape(-1).long(), ignore_index=-100, reduction="sum")
    return loss, aux_total

"""Dispatch for the native (tcgen05) flash-attention kernels.

The kernels are causal with an optional per-query LOWER BOUND: query ``t`` attends keys ``lo[t] <= k <= t``.  Packed
documents (``lo`` = first position of the query's document), sliding windows (``lo = t - window + 1``) and their
combination (the maximum of the two) are all expressed through that one int32 array, which is non-decreasing along a
sequence; the backward pass additionally gets, per 128-key tile, the end of the query range that can still see it.
Both arrays depend only on the batch's document ids and the layer's window, so they are built once per micro-batch and
window and shared by every layer (``ExecContext.attn_bounds``).

Parity: csrc/src/runtime/attention/backend_flash_varlen.cpp:41-63 (cu_seqlens from position-id resets),
attention_custom.cu (sliding window).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def native_supported(attrs, qkv, ctx) -> bool:
    ext_has = hasattr(_ext_mod(), "flash_attn_fwd")
    return (ext_has and attrs["head_dim"] == 128 and attrs.get("causal", True) and not attrs.get("sinks", False)
            and qkv.dtype == torch.bfloat16 and qkv.shape[1] % 128 == 0)


def _ext_mod():
    from . import ext

    return ext()


def lower_bounds(doc_ids: Optional[torch.Tensor], window: int, B: int, T: int, device) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
    """(lo [B, T] int32, kv_qend [B, T/128] int32) for a batch of packed documents and / or a sliding window; None when plain
    causal attention applies.  Pure tensor code (no host sync); also the CPU oracle of the kernels' masking rule."""
    if doc_ids is None and not window:
        return None
    idx = torch.arange(T, device=device, dtype=torch.int32)
    lo = torch.zeros(B, T, dtype=torch.int32, device=device)
    if doc_ids is not None:
        d = doc_ids.to(device)
        first = torch.ones(B, T, dtype=torch.bool, device=device)
        first[:, 1:] = d[:, 1:] != d[:, :-1]
        lo = torch.cummax(torch.where(first, idx.expand(B, T), torch.zeros_like(lo)), dim=1).values.to(torch.int32)
    if window:
        lo = torch.maximum(lo, (idx - (int(window) - 1)).clamp_min(0).expand(B, T))
    lo = lo.contiguous()
    k_last = (torch.arange(T // 128, device=device, dtype=torch.int32) * 128 + 127).expand(B, T // 128).contiguous()
    seen = torch.searchsorted(lo, k_last, right=True)          # number of queries whose lower bound is <= the tile's last key
    kv_qend = ((seen + 63) // 64).to(torch.int32).contiguous()
    return lo, kv_qend


def _bounds(attrs, qkv, ctx):
    window = int(attrs.get("window", 0) or 0)
    doc_ids = getattr(ctx, "doc_ids", None)
    if doc_ids is None and not window:
        return None
    cache = getattr(ctx, "attn_bounds", None)
    if cache is None:
        cache = ctx.attn_bounds = {}
    key = (window, qkv.shape[1])
    if key not in cache:
        cache[key] = lower_bounds(doc_ids, window, qkv.shape[0], qkv.shape[1], qkv.device)
    return cache[key]


def forward(ext, attrs, qkv, ctx):
    Hq, Hkv, D = attrs["num_q_heads"], attrs["num_kv_heads"], attrs["head_dim"]
    scale = attrs.get("softmax_scale") or 1.0 / math.sqrt(D)
    b = _bounds(attrs, qkv, ctx)
    att, lse = ext.flash_attn_fwd(qkv, Hq, Hkv, float(scale), b[0] if b is not None else None)
    return att, lse


def backward(ext, attrs, d_att, qkv, att, lse, ctx):
    Hq, Hkv, D = attrs["num_q_heads"], attrs["num_kv_heads"], attrs["head_dim"]
    scale = attrs.get("softmax_scale") or 1.0 / math.sqrt(D)
    b = _bounds(attrs, qkv, ctx)
    lo, qend = b if b is not None else (None, None)
    return (ext.flash_attn_bwd(d_att.contiguous(), qkv, att, lse, Hq, Hkv, float(scale), lo, qend),)

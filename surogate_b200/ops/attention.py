"""Dispatch for the native (tcgen05) flash-attention kernels."""
from __future__ import annotations

import math

import torch


def native_supported(attrs, qkv, ctx) -> bool:
    ext_has = hasattr(_ext_mod(), "flash_attn_fwd")
    return (ext_has and attrs["head_dim"] == 128 and attrs.get("causal", True) and not attrs.get("window", 0)
            and qkv.dtype == torch.bfloat16 and ctx.doc_ids is None and qkv.shape[1] % 128 == 0)


def _ext_mod():
    from . import ext

    return ext()


def forward(ext, attrs, qkv, ctx):
    B, T = qkv.shape[:2]
    Hq, Hkv, D = attrs["num_q_heads"], attrs["num_kv_heads"], attrs["head_dim"]
    scale = attrs.get("softmax_scale") or 1.0 / math.sqrt(D)
    att, lse = ext.flash_attn_fwd(qkv, Hq, Hkv, float(scale))
    return att, lse


def backward(ext, attrs, d_att, qkv, att, lse, ctx):
    Hq, Hkv, D = attrs["num_q_heads"], attrs["num_kv_heads"], attrs["head_dim"]
    scale = attrs.get("softmax_scale") or 1.0 / math.sqrt(D)
    return (ext.flash_attn_bwd(d_att.contiguous(), qkv, att, lse, Hq, Hkv, float(scale)),)

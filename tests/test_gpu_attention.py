"""tcgen05 flash attention against an fp32 PyTorch reference (causal, grouped-query heads, head_dim 128)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref(qkv, Hq, Hkv, scale):
    B, T, _ = qkv.shape
    D = 128
    x = qkv.float().view(B, T, Hq + 2 * Hkv, D)
    q, k, v = x[:, :, :Hq], x[:, :, Hq:Hq + Hkv], x[:, :, Hq + Hkv:]
    G = Hq // Hkv
    q = q.permute(0, 2, 1, 3)
    k = k.permute(0, 2, 1, 3).repeat_interleave(G, 1)
    v = v.permute(0, 2, 1, 3).repeat_interleave(G, 1)
    s = q @ k.transpose(-1, -2) * scale
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.softmax(s, -1) @ v
    return o.permute(0, 2, 1, 3).reshape(B, T, Hq * D), lse.permute(0, 2, 1)


@pytest.mark.parametrize("B,T,Hq,Hkv", [(1, 128, 1, 1), (2, 256, 4, 2), (1, 1024, 8, 2), (2, 512, 2, 2)])
def test_flash_attention_forward(B, T, Hq, Hkv):
    from surogate_b200.ops import check_device_errors, ext

    e = ext()
    torch.manual_seed(B * T + Hq)
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * 128, device=DEV).bfloat16()
    qkv[:, :, : Hq * 128] *= 2.0   # sharper scores: exercises the running-max rescale
    scale = 1.0 / math.sqrt(128)
    out, lse = e.flash_attn_fwd_raw(qkv, Hq, Hkv, scale, e.error_flag_tensor())
    torch.cuda.synchronize()
    check_device_errors()
    ro, rl = _ref(qkv, Hq, Hkv, scale)
    assert torch.allclose(lse, rl, rtol=2e-3, atol=2e-3), (lse - rl).abs().max()
    err = ((out.float() - ro).norm() / ro.norm()).item()
    assert err < 8e-3, err


@pytest.mark.parametrize("B,T,Hq,Hkv", [(1, 128, 1, 1), (2, 256, 4, 2), (1, 512, 8, 2)])
def test_flash_attention_backward(B, T, Hq, Hkv):
    from surogate_b200.ops import check_device_errors, ext

    e = ext()
    torch.manual_seed(7 + T)
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * 128, device=DEV).bfloat16()
    scale = 1.0 / math.sqrt(128)
    out, lse = e.flash_attn_fwd(qkv, Hq, Hkv, scale)
    d_out = torch.randn_like(out)
    d_qkv = e.flash_attn_bwd(d_out, qkv, out, lse, Hq, Hkv, scale)
    torch.cuda.synchronize()
    check_device_errors()
    x = qkv.float().requires_grad_(True)
    ro, _ = _ref(x, Hq, Hkv, scale)
    ro.backward(d_out.float())
    g = x.grad
    D = 128
    for name, lo, hi in [("dq", 0, Hq * D), ("dk", Hq * D, (Hq + Hkv) * D), ("dv", (Hq + Hkv) * D, (Hq + 2 * Hkv) * D)]:
        a, b = d_qkv[..., lo:hi].float(), g[..., lo:hi]
        err = ((a - b).norm() / b.norm()).item()
        assert err < 1.5e-2, (name, err)

"""tcgen05 flash attention against an fp32 PyTorch reference (causal, grouped-query heads, head_dim 128; packed documents and
sliding windows through the per-query lower bound)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
D = 128


def _ref(qkv, Hq, Hkv, scale, lo=None):
    """fp32 attention, one KV head group at a time (keeps the [T, T] score matrices of the large cases in memory bounds)."""
    B, T, _ = qkv.shape
    x = qkv.view(B, T, Hq + 2 * Hkv, D)
    G = Hq // Hkv
    i = torch.arange(T, device=qkv.device)
    ok = (i[:, None] >= i[None, :]).expand(B, T, T)
    if lo is not None:
        ok = ok & (i[None, None, :] >= lo.long()[:, :, None])
    outs, lses = [], []
    for hk in range(Hkv):
        q = x[:, :, hk * G:(hk + 1) * G].float().permute(0, 2, 1, 3)
        k = x[:, :, Hq + hk].float()[:, None]
        v = x[:, :, Hq + Hkv + hk].float()[:, None]
        s = (q @ k.transpose(-1, -2) * scale).masked_fill(~ok[:, None], float("-inf"))
        lses.append(torch.logsumexp(s, -1))
        outs.append(torch.softmax(s, -1) @ v)
    o = torch.cat(outs, 1)
    return o.permute(0, 2, 1, 3).reshape(B, T, Hq * D), torch.cat(lses, 1).permute(0, 2, 1)


def _packed_lo(B, T, window=0, docs=True, seed=0):
    """Document ids with random boundaries (not aligned to the kernels' 64 / 128 tiles) and the bounds derived from them."""
    from surogate_b200.ops.attention import lower_bounds

    g = torch.Generator().manual_seed(seed)
    doc_ids = None
    if docs:
        cuts = torch.zeros(B, T, dtype=torch.int32)
        for b in range(B):
            n = int(torch.randint(2, 7, (1,), generator=g))
            pos = torch.randint(1, T, (n,), generator=g)
            cuts[b, pos] = 1
        cuts[0, 64] = 1
        cuts[0, min(T - 1, 128)] = 1            # boundaries exactly on tile edges too
        doc_ids = torch.cumsum(cuts, 1).to(DEV)
    return lower_bounds(doc_ids, window, B, T, torch.device(DEV))


def _check_fwd(qkv, Hq, Hkv, lo=None, tol=8e-3):
    from surogate_b200.ops import check_device_errors, ext

    e = ext()
    scale = 1.0 / math.sqrt(D)
    out, lse = e.flash_attn_fwd(qkv, Hq, Hkv, scale, lo)
    torch.cuda.synchronize()
    check_device_errors()
    ro, rl = _ref(qkv, Hq, Hkv, scale, lo)
    assert torch.allclose(lse, rl, rtol=2e-3, atol=2e-3), (lse - rl).abs().max()
    err = ((out.float() - ro).norm() / ro.norm()).item()
    assert err < tol, err
    return out, lse


def _check_bwd(qkv, Hq, Hkv, bounds=None, tol=1.5e-2):
    from surogate_b200.ops import check_device_errors, ext

    e = ext()
    scale = 1.0 / math.sqrt(D)
    lo, qend = bounds if bounds is not None else (None, None)
    out, lse = e.flash_attn_fwd(qkv, Hq, Hkv, scale, lo)
    d_out = torch.randn_like(out)
    d_qkv = e.flash_attn_bwd(d_out, qkv, out, lse, Hq, Hkv, scale, lo, qend)
    torch.cuda.synchronize()
    check_device_errors()
    x = qkv.float().requires_grad_(True)
    ro, _ = _ref(x, Hq, Hkv, scale, lo)
    ro.backward(d_out.float())
    g = x.grad
    for name, a, z in [("dq", 0, Hq * D), ("dk", Hq * D, (Hq + Hkv) * D), ("dv", (Hq + Hkv) * D, (Hq + 2 * Hkv) * D)]:
        u, v = d_qkv[..., a:z].float(), g[..., a:z]
        err = ((u - v).norm() / v.norm()).item()
        assert err < tol, (name, err)


@pytest.mark.parametrize("B,T,Hq,Hkv", [(1, 128, 1, 1), (2, 256, 4, 2), (1, 1024, 8, 2), (2, 512, 2, 2)])
def test_flash_attention_forward(B, T, Hq, Hkv):
    torch.manual_seed(B * T + Hq)
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    qkv[:, :, : Hq * D] *= 2.0   # sharper scores: exercises the running-max rescale
    _check_fwd(qkv, Hq, Hkv)


@pytest.mark.parametrize("B,T,Hq,Hkv", [(1, 128, 1, 1), (2, 256, 4, 2), (1, 512, 8, 2)])
def test_flash_attention_backward(B, T, Hq, Hkv):
    torch.manual_seed(7 + T)
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    _check_bwd(qkv, Hq, Hkv)


@pytest.mark.parametrize("B,T,Hq,Hkv", [(2, 4096, 32, 8), (1, 8192, 40, 8)])
def test_flash_attention_at_the_benchmark_shapes(B, T, Hq, Hkv):
    """The head counts and sequence lengths the Qwen3-8B and Qwen3-14B configurations run, forward and backward."""
    torch.manual_seed(T)
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    _check_fwd(qkv, Hq, Hkv)
    _check_bwd(qkv, Hq, Hkv)


@pytest.mark.parametrize("B,T,Hq,Hkv,window,docs", [(2, 512, 4, 2, 0, True), (1, 1024, 8, 2, 200, False), (2, 1024, 4, 1, 128, True),
                                                    (1, 2048, 4, 4, 3, False), (2, 4096, 8, 2, 0, True), (1, 4096, 8, 2, 1024, True)])
def test_flash_attention_packed_documents_and_windows(B, T, Hq, Hkv, window, docs):
    """Per-query lower bounds: queries attend only inside their own document and / or the last `window` keys; tiles that no query of
    a block can see are skipped by the kernels, so boundaries inside and on tile edges are both covered."""
    torch.manual_seed(T + window)
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    qkv[:, :, : Hq * D] *= 1.5
    bounds = _packed_lo(B, T, window, docs, seed=T + window)
    lo, qend = bounds
    i = torch.arange(T, device=DEV)
    assert bool((lo[:, 1:] >= lo[:, :-1]).all()) and bool((lo <= i).all())
    assert bool((qend >= 2 * (torch.arange(T // 128, device=DEV) + 1)).all()) and int(qend.max()) <= T // 64
    _check_fwd(qkv, Hq, Hkv, lo)
    _check_bwd(qkv, Hq, Hkv, bounds)


def test_packed_batch_trains_like_the_masked_fp32_path():
    """One packed batch (position ids reset inside the rows) and one sliding-window model through the trainer on the CUDA backend:
    loss and gradient norm equal the PyTorch backend, whose attention applies the explicit document / window mask."""
    import numpy as np

    from surogate_b200.runtime.trainer import Trainer, TrainerConfig

    rng = np.random.default_rng(0)
    T = 256
    tok = rng.integers(0, 512, (2, T + 1)).astype(np.int32)
    pos = np.stack([np.concatenate([np.arange(100), np.arange(60), np.arange(96)]), np.concatenate([np.arange(128), np.arange(128)])]).astype(np.int32)
    for window in (0, 96):
        model = dict(architecture="Qwen3ForCausalLM", vocab_size=512, d_model=256, n_layers=2, num_query_heads=2, num_kv_heads=1, head_size=128, d_ff=512,
                     tie_word_embeddings=True)
        if window:
            model["sliding_window"] = window
        res = {}
        for backend in ("cuda", "ref"):
            cfg = TrainerConfig(model=model, batch_size=2, seq_len=T, recipe="bf16", optimizer="adamw", learning_rate=1e-3, backend=backend)
            tr = Trainer(cfg, device=torch.device("cuda:0"))
            tr.init_weights(seed=0)
            res[backend] = tr.step(tok[:, :-1], tok[:, 1:], position_ids=pos)
        assert abs(res["cuda"]["loss"] - res["ref"]["loss"]) < 2e-2 * res["ref"]["loss"], (window, res)
        assert abs(res["cuda"]["norm"] - res["ref"]["norm"]) < 5e-2 * res["ref"]["norm"], (window, res)
        # and the mask matters: without the position resets the loss is a different number
        cfg = TrainerConfig(model=model, batch_size=2, seq_len=T, recipe="bf16", optimizer="adamw", learning_rate=1e-3, backend="ref")
        tr = Trainer(cfg, device=torch.device("cuda:0"))
        tr.init_weights(seed=0)
        plain = tr.step(tok[:, :-1], tok[:, 1:])
        assert abs(plain["loss"] - res["ref"]["loss"]) > 1e-4

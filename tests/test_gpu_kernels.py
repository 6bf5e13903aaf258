"""Numerics of each hand-written sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def ext():
    from surogate_b200.ops import ext as load

    return load()


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _check_flag():
    from surogate_b200.ops import check_device_errors

    check_device_errors()


# ----------------------------------------------------------------------------- GEMM
GEMM_SHAPES = [(256, 256, 128), (128, 128, 64), (384, 512, 320), (300, 264, 200), (1024, 1536, 1024), (136, 8, 64), (4096, 512, 2048)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_bf16(ext, M, N, K, a_mn, b_mn):
    from surogate_b200.runtime.ops_cuda import gemm

    if (a_mn and M % 8) or (b_mn and N % 8) or K % 8:
        pytest.skip("row stride must be a multiple of 16 bytes")
    torch.manual_seed(M + N + K)
    A = torch.randn(M, K, device=DEV)
    B = torch.randn(N, K, device=DEV)
    a = (A.t().contiguous() if a_mn else A).bfloat16()
    b = (B.t().contiguous() if b_mn else B).bfloat16()
    ref = (a.t() if a_mn else a).float() @ (b.t() if b_mn else b).float().t()
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    _check_flag()
    assert _rel_err(out, ref) < 6e-3, _rel_err(out, ref)


PAIR_SHAPES = [(256, 256, 128), (512, 768, 320), (300, 264, 200), (1024, 1536, 1024), (2048, 1000, 4096), (4096, 512, 2048), (128, 520, 64)]


@pytest.mark.parametrize("M,N,K", PAIR_SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("fp8", [False, True])
def test_gemm_cta_pair(ext, M, N, K, a_mn, b_mn, fp8):
    """The cta_group::2 kernel (256 x 256 tile per two-CTA cluster, TMA-store epilogue), forced with tile_n=512: every operand
    layout, bf16 and FP8, ragged edges in M, N and K, bf16 and fp32 outputs, fp32 accumulation (TMA add) and bf16 accumulation."""
    from surogate_b200.runtime.ops_cuda import gemm

    es = 1 if fp8 else 2
    if (a_mn and M * es % 16) or (b_mn and N * es % 16) or K * es % 16 or N % 8:
        pytest.skip("row stride must be a multiple of 16 bytes")
    torch.manual_seed(M + N + K)
    A = torch.randn(M, K, device=DEV)
    B = torch.randn(N, K, device=DEV)
    dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    a = (A.t().contiguous() if a_mn else A).to(dt)
    b = (B.t().contiguous() if b_mn else B).to(dt)
    ref = (a.float().t() if a_mn else a.float()) @ (b.float().t() if b_mn else b.float()).t()
    kw = dict(scale_a=torch.tensor([0.5], device=DEV), scale_b=torch.tensor([2.0], device=DEV)) if fp8 else {}
    amax = torch.zeros(1, device=DEV)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, tile_n=512, amax_out=amax, **kw)
    torch.cuda.synchronize()
    _check_flag()
    assert _rel_err(out, ref) < 6e-3, _rel_err(out, ref)
    assert abs(amax.item() - out.float().abs().max().item()) <= 0.01 * amax.item()
    out32 = gemm(a, b, a_mn=a_mn, b_mn=b_mn, tile_n=512, out_dtype=torch.float32, **kw)
    assert _rel_err(out32, ref) < 1e-4 if not fp8 else _rel_err(out32, ref) < 1e-4
    base = torch.randn(M, N, device=DEV)
    acc32 = base.clone()
    gemm(a, b, acc32, a_mn=a_mn, b_mn=b_mn, tile_n=512, accumulate=True, alpha=0.5, **kw)
    assert _rel_err(acc32, base + 0.5 * ref) < 1e-4
    acc16 = base.bfloat16()
    ref16 = acc16.float() + ref
    gemm(a, b, acc16, a_mn=a_mn, b_mn=b_mn, tile_n=512, accumulate=True, **kw)
    assert _rel_err(acc16, ref16) < 6e-3
    # a view into a wider buffer: the store must not touch the columns next to it
    wide = torch.zeros(M, N + 64, device=DEV, dtype=torch.bfloat16)
    gemm(a, b, wide[:, 32:32 + N], a_mn=a_mn, b_mn=b_mn, tile_n=512, **kw)
    assert _rel_err(wide[:, 32:32 + N], ref) < 6e-3
    assert wide[:, :32].abs().max() == 0 and wide[:, 32 + N:].abs().max() == 0
    torch.cuda.synchronize()
    _check_flag()


def test_gemm_accumulate_fp32_and_alpha(ext):
    from surogate_b200.runtime.ops_cuda import gemm

    M, N, K = 512, 384, 256
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = torch.randn(N, K, device=DEV).bfloat16()
    base = torch.randn(M, N, device=DEV)
    out = base.clone()
    gemm(a, b, out, accumulate=True, alpha=0.5)
    ref = base + 0.5 * (a.float() @ b.float().t())
    assert _rel_err(out, ref) < 1e-4
    out16 = base.bfloat16()
    ref16 = out16.float() + a.float() @ b.float().t()
    gemm(a, b, out16, accumulate=True)
    assert _rel_err(out16, ref16) < 6e-3
    # strided output / strided inputs (views into wider buffers)
    wide = torch.zeros(M, N + 64, device=DEV, dtype=torch.bfloat16)
    gemm(a, b, wide[:, 32:32 + N])
    assert _rel_err(wide[:, 32:32 + N], a.float() @ b.float().t()) < 6e-3
    assert wide[:, :32].abs().max() == 0 and wide[:, 32 + N:].abs().max() == 0
    _check_flag()


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (384, 512, 384), (1024, 768, 2048), (272, 264, 144)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("a_e5m2", [False, True])
def test_gemm_fp8(ext, M, N, K, a_mn, b_mn, a_e5m2):
    from surogate_b200.runtime.ops_cuda import gemm

    if (a_mn and M % 16) or (b_mn and N % 16) or K % 16:
        pytest.skip("row stride must be a multiple of 16 bytes")
    torch.manual_seed(1)
    A = torch.randn(M, K, device=DEV)
    B = torch.randn(N, K, device=DEV)
    a = (A.t().contiguous() if a_mn else A).to(torch.float8_e5m2 if a_e5m2 else torch.float8_e4m3fn)
    b = (B.t().contiguous() if b_mn else B).to(torch.float8_e4m3fn)
    sa = torch.tensor([0.5], device=DEV)
    sb = torch.tensor([2.5], device=DEV)
    ref = 1.25 * ((a.float().t() if a_mn else a.float()) @ (b.float().t() if b_mn else b.float()).t())
    amax = torch.zeros(1, device=DEV)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, scale_a=sa, scale_b=sb, amax_out=amax)
    torch.cuda.synchronize()
    _check_flag()
    assert _rel_err(out, ref) < 6e-3, _rel_err(out, ref)
    assert abs(amax.item() - out.float().abs().max().item()) <= 0.01 * amax.item()


# ----------------------------------------------------------------------------- norms
@pytest.mark.parametrize("C", [1024, 4096, 5120])
def test_rmsnorm_fwd_bwd(ext, C):
    rows = 333
    x = torch.randn(rows, C, device=DEV).bfloat16()
    r = torch.randn(rows, C, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(C, device=DEV)).bfloat16()
    res, y, rstd, _ = ext.rmsnorm_fwd(x, r, w, 1e-6, True, None, None, False)
    rf = (x.float() + r.float()).bfloat16().float()
    ref_rstd = torch.rsqrt(rf.pow(2).mean(-1) + 1e-6)
    assert torch.equal(res, rf.bfloat16())
    assert torch.allclose(rstd, ref_rstd, rtol=1e-4)
    assert _rel_err(y, rf * ref_rstd[:, None] * w.float()) < 5e-3
    dy = torch.randn(rows, C, device=DEV).bfloat16()
    dres = torch.randn(rows, C, device=DEV).bfloat16()
    dx, dw = ext.rmsnorm_bwd(dy, res, w, rstd, dres)
    xhat = rf * ref_rstd[:, None]
    dn = dy.float() * w.float()
    ref_dx = ref_rstd[:, None] * (dn - xhat * (dn * xhat).mean(-1, keepdim=True)) + dres.float()
    assert _rel_err(dx, ref_dx) < 5e-3
    assert _rel_err(dw, (dy.float() * xhat).sum(0)) < 1e-4
    # fp8 output with scale and abs-max
    scale = torch.tensor([3.0], device=DEV)
    amax = torch.zeros(1, device=DEV)
    _, _, _, y8 = ext.rmsnorm_fwd(x, r, w, 1e-6, False, scale, amax, True)
    yref = rf * ref_rstd[:, None] * w.float()
    assert _rel_err(y8.float() / 3.0, yref) < 0.05
    assert abs(amax.item() - yref.abs().max().item()) < 0.02 * amax.item()


def test_swiglu(ext):
    rows, M = 517, 3072
    x = torch.randn(rows, 2 * M, device=DEV).bfloat16()
    y = ext.swiglu_fwd(x, True, None, None, False)[0]
    up, gate = x[:, :M].float(), x[:, M:].float()
    assert _rel_err(y, torch.nn.functional.silu(gate) * up) < 5e-3
    dy = torch.randn(rows, M, device=DEV).bfloat16()
    dx = ext.swiglu_bwd(dy, x)
    s = torch.sigmoid(gate)
    ref = torch.cat([dy.float() * gate * s, dy.float() * up * s * (1 + gate * (1 - s))], -1)
    assert _rel_err(dx, ref) < 5e-3


@pytest.mark.parametrize("B,T,Hq,Hkv", [(2, 96, 8, 2), (1, 50, 3, 1), (1, 300, 32, 8), (2, 33, 5, 5)])
def test_qk_norm_rope(ext, B, T, Hq, Hkv):
    """Even and odd head counts (a half-warp without a head of its own still takes part in the shuffles), the benchmark's 32 / 8."""
    from surogate_b200.dsl.ir import OpNode
    from surogate_b200.runtime.ops_ref import RefOps

    D = 128
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    qw = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16()
    kw = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16()
    pos = torch.arange(T, device=DEV, dtype=torch.int32)[None].repeat(B, 1).contiguous()
    attrs = dict(num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D, eps=1e-6, rope_theta=1e6, rotary_dim=D)
    ref = RefOps()
    op = OpNode("qkv_qk_norm_rope", [], [], attrs)
    r_out, r_q, r_k = ref.qkv_qk_norm_rope(None, op, qkv.float(), qw.float(), kw.float(), pos)
    out, q_rstd, k_rstd = ext.qk_norm_rope_fwd(qkv, qw, kw, pos, Hq, Hkv, D, 1e-6, 1e6)
    assert _rel_err(out, r_out) < 5e-3
    assert torch.allclose(q_rstd, r_q, rtol=1e-4) and torch.allclose(k_rstd, r_k, rtol=1e-4)
    dy = torch.randn_like(qkv)
    r_dx, r_dq, r_dk = ref.qkv_qk_norm_rope_backward(None, op, dy.float(), qkv.float(), qw.float(), kw.float(), r_q, r_k, pos)
    dx, dqw, dkw = ext.qk_norm_rope_bwd(dy, qkv, qw, kw, q_rstd, k_rstd, pos, Hq, Hkv, D, 1e-6, 1e6)
    assert _rel_err(dx, r_dx) < 5e-3
    assert _rel_err(dqw, r_dq) < 2e-3 and _rel_err(dkw, r_dk) < 2e-3
    # without qk-norm (Llama-style)
    out2, _, _ = ext.qk_norm_rope_fwd(qkv, None, None, pos, Hq, Hkv, D, 1e-6, 1e4)
    attrs2 = dict(attrs, rope_theta=1e4)
    r2, _, _ = ref.qkv_qk_norm_rope(None, OpNode("x", [], [], attrs2), qkv.float(), None, None, pos)
    assert _rel_err(out2, r2) < 5e-3


def test_qk_norm_rope_multi_axis_positions(ext):
    """(t, h, w) rotary positions: frequency j reads the height row if j % 3 == 1 and j < 3 * sec_h, the width row if
    j % 3 == 2 and j < 3 * sec_w, else the temporal row; forward and backward against the PyTorch op."""
    from types import SimpleNamespace

    from surogate_b200.dsl.ir import OpNode
    from surogate_b200.runtime.ops_ref import RefOps

    B, T, Hq, Hkv, D = 2, 64, 4, 2, 128
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    qw = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16()
    kw = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16()
    pos3 = torch.stack([torch.arange(T, device=DEV)[None].repeat(B, 1), torch.randint(0, 40, (B, T), device=DEV), torch.randint(0, 40, (B, T), device=DEV)]).to(torch.int32)
    attrs = dict(num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D, eps=1e-6, rope_theta=5e6, rotary_dim=D, mrope_section=[24, 20, 20])
    ctx = SimpleNamespace(extras={"mrope_position_ids": pos3})
    op = OpNode("qkv_qk_norm_rope", [], [], attrs)
    ref = RefOps()
    r_out, r_q, r_k = ref.qkv_qk_norm_rope(ctx, op, qkv.float(), qw.float(), kw.float(), pos3[0])
    out, q_rstd, k_rstd = ext.qk_norm_rope_fwd(qkv, qw, kw, pos3.contiguous(), Hq, Hkv, D, 1e-6, 5e6, 20, 20)
    assert _rel_err(out, r_out) < 5e-3
    plain, _, _ = ext.qk_norm_rope_fwd(qkv, qw, kw, pos3[0].contiguous(), Hq, Hkv, D, 1e-6, 5e6)
    assert _rel_err(plain, r_out) > 0.05  # the height / width rows matter
    dy = torch.randn_like(qkv)
    r_dx, r_dq, r_dk = ref.qkv_qk_norm_rope_backward(ctx, op, dy.float(), qkv.float(), qw.float(), kw.float(), r_q, r_k, pos3[0])
    dx, dqw, dkw = ext.qk_norm_rope_bwd(dy, qkv, qw, kw, q_rstd, k_rstd, pos3.contiguous(), Hq, Hkv, D, 1e-6, 5e6, 20, 20)
    assert _rel_err(dx, r_dx) < 5e-3 and _rel_err(dqw, r_dq) < 2e-3 and _rel_err(dkw, r_dk) < 2e-3


def test_embedding(ext):
    V, C, n = 1000, 512, 4096
    table = torch.randn(V, C, device=DEV).bfloat16()
    tok = torch.randint(0, V, (4, n // 4), device=DEV, dtype=torch.int32)
    out = ext.embedding_fwd(tok, table)
    assert torch.equal(out, table[tok.long()])
    dout = torch.randn(4, n // 4, C, device=DEV).bfloat16()
    g = torch.zeros(V, C, device=DEV, dtype=torch.float32)
    ext.embedding_bwd(tok, dout, g)
    ref = torch.zeros(V, C, device=DEV).index_add_(0, tok.reshape(-1).long(), dout.reshape(-1, C).float())
    assert _rel_err(g, ref) < 1e-5
    # the default (sorted, no atomics) is bit-reproducible, also into a bf16 table and with a heavily repeated id; the atomic variant agrees
    tok[0, :700] = 7
    ref = torch.zeros(V, C, device=DEV).index_add_(0, tok.reshape(-1).long(), dout.reshape(-1, C).float())
    runs = []
    for _ in range(2):
        gb = torch.zeros(V, C, device=DEV, dtype=torch.bfloat16)
        ext.embedding_bwd(tok, dout, gb)
        runs.append(gb)
    assert torch.equal(runs[0], runs[1]) and _rel_err(runs[0], ref) < 4e-3
    ga = torch.zeros(V, C, device=DEV, dtype=torch.float32)
    ext.embedding_bwd(tok, dout, ga, False)
    assert _rel_err(ga, ref) < 1e-5


def test_cross_entropy(ext):
    rows, V = 257, 151936 // 8
    logits = (3 * torch.randn(rows, V, device=DEV)).bfloat16()
    tgt = torch.randint(0, V, (rows,), device=DEV, dtype=torch.int32)
    tgt[::7] = -100
    ref_logits = logits.float().requires_grad_(True)
    ref_loss = torch.nn.functional.cross_entropy(ref_logits, tgt.long(), ignore_index=-100, reduction="none")
    (ref_loss.sum() * 0.25).backward()
    scale = torch.tensor([0.5], device=DEV)
    work = logits.clone()
    loss = ext.cross_entropy_fwd_bwd(work, tgt, scale, 0.5, True)
    assert torch.allclose(loss, ref_loss.detach(), rtol=1e-3, atol=1e-3)
    assert _rel_err(work, ref_logits.grad) < 1e-2
    assert work[::7].abs().max() == 0


def test_quantize_fp8_and_sumsq(ext):
    x = (5 * torch.randn(1 << 20, device=DEV)).bfloat16()
    scale = torch.tensor([4.0], device=DEV)
    amax = torch.zeros(1, device=DEV)
    q = ext.quantize_fp8(x, scale, amax, False)
    assert torch.equal(q.view(torch.uint8), (x.float() * 4).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8))
    assert amax.item() == x.float().abs().max().item()
    q2 = ext.quantize_fp8(x, scale, None, True)
    assert torch.equal(q2.view(torch.uint8), (x.float() * 4).to(torch.float8_e5m2).view(torch.uint8))
    assert abs(ext.sumsq(x).item() / x.float().pow(2).sum().item() - 1) < 1e-4
    xf = torch.randn(12345, device=DEV)
    assert abs(ext.sumsq(xf).item() / xf.pow(2).sum().item() - 1) < 1e-5


def test_adamw_kernels(ext):
    n = 100000 - 100000 % 32
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV) * 0.1
    mask = (torch.arange(n, device=DEV) % 3 != 0).to(torch.uint8)
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
    p_ref, m_ref, v_ref = p.clone(), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    p32, m, v = p.clone(), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    p8 = p.clone()
    m8, v8 = torch.zeros(n, dtype=torch.int8, device=DEV), torch.zeros(n, dtype=torch.uint8, device=DEV)
    ng = (n + 31) // 32
    ms, vs = torch.zeros(ng, dtype=torch.float16, device=DEV), torch.zeros(ng, dtype=torch.float16, device=DEV)
    for step in range(1, 6):
        gs = g * (1 + 0.1 * step)
        hp = torch.tensor([lr, b1, b2, eps, wd, 1 - b1 ** step, 1 - b2 ** step, 1.0], device=DEV)
        m_ref = b1 * m_ref + (1 - b1) * gs
        v_ref = b2 * v_ref + (1 - b2) * gs * gs
        p_ref = p_ref * (1 - lr * wd * mask) - lr * (m_ref / (1 - b1 ** step)) / ((v_ref / (1 - b2 ** step)).sqrt() + eps)
        ext.adamw_step(p32, gs, m, v, mask, hp)
        ext.adamw8_step(p8, gs, m8, v8, ms, vs, mask, hp)
    assert _rel_err(p32, p_ref) < 1e-5
    # 8-bit state: updates stay close to the fp32-state trajectory
    assert _rel_err(p8 - p, p_ref - p) < 0.1
    # bf16 params / grads variant
    pb = p.bfloat16()
    ext.adamw_step(pb, g.bfloat16(), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV), None,
                   torch.tensor([lr, b1, b2, eps, 0.0, 1 - b1, 1 - b2, 1.0], device=DEV))
    assert torch.isfinite(pb.float()).all()


def test_adamw_8bit_kernel_matches_the_pytorch_twin_code_for_code(ext):
    """Three steps of the 8-bit kernel against the PyTorch statement of the same state encoding (optim/adamw.py): the parameters
    agree to fp32 rounding of the approximated divisions, the int8 / uint8 codes are equal except for values that sit on a rounding
    boundary (off by one at most), the fp16 group scales are equal or one fp16 step apart."""
    from surogate_b200.optim.adamw import _softsign_dequant_reference, _softsign_quant_reference

    torch.manual_seed(3)
    n = 32 * 4096
    lr, b1, b2, eps, wd = 3e-3, 0.9, 0.95, 1e-8, 0.1
    for pdt, gdt in ((torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)):
        p = torch.randn(n, device=DEV).to(pdt)
        blocks = (torch.arange(n // 128, device=DEV) % 2 == 0).to(torch.uint8)
        mask = blocks.repeat_interleave(128).float()
        m8, v8 = torch.zeros(n, dtype=torch.int8, device=DEV), torch.zeros(n, dtype=torch.uint8, device=DEV)
        ms, vs = torch.zeros(n // 32, dtype=torch.float16, device=DEV), torch.zeros(n // 32, dtype=torch.float16, device=DEV)
        rm8, rv8, rms, rvs, rp = m8.clone(), v8.clone(), ms.clone(), vs.clone(), p.clone()
        for step in range(1, 4):
            g = (torch.randn(n, device=DEV) * 0.05 * torch.rand(n, device=DEV).pow(4)).to(gdt)
            bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
            hp = torch.tensor([lr, b1, b2, eps, wd, bc1, bc2, 0.7], device=DEV)
            ext.adamw8_step(p, g, m8, v8, ms, vs, blocks, hp)
            m, v = _softsign_dequant_reference(rm8, rv8, rms, rvs)
            gf = g.float() * 0.7
            m = b1 * m + (1 - b1) * gf
            v = b2 * v + (1 - b2) * gf * gf
            pn = rp.float() * (1 - lr * wd * mask) - lr * (m / bc1) / ((v / bc2).sqrt() + eps)
            upd_ref, upd = pn - rp.float(), p.float() - rp.float()
            rp = pn.to(pdt)
            rm8, rv8, rms, rvs = _softsign_quant_reference(m, v)
            if pdt == torch.float32:
                assert _rel_err(upd, upd_ref) < 2e-3, (step, _rel_err(upd, upd_ref))
            else:
                assert (p.float() - rp.float()).abs().max() <= 2 * 2 ** -7 * rp.float().abs().max()
            dm = (m8.int() - rm8.int()).abs()
            dv = (v8.int() - rv8.int()).abs()
            assert int(dm.max()) <= 1 and int(dv.max()) <= 1, (int(dm.max()), int(dv.max()))
            assert float((dm > 0).float().mean()) < 0.03 and float((dv > 0).float().mean()) < 0.03
            assert float((ms.float() - rms.float()).abs().max() / rms.float().abs().max()) < 2e-3
            # the next step starts from the kernel's own state on both sides, so differences do not accumulate
            rm8, rv8, rms, rvs, rp = m8.clone(), v8.clone(), ms.clone(), vs.clone(), p.clone()
    _check_flag()


# ----------------------------------------------------------------------------- MoE
def test_moe_softmax_topk(ext):
    tokens, E, K = 1000, 128, 8
    logits = torch.randn(tokens, E, device=DEV)
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    psum = torch.zeros(E, device=DEV)
    lse = torch.zeros(1, device=DEV)
    w, idx, probs = ext.moe_softmax_topk(logits, K, True, counts, psum, lse, True)
    ref_p = torch.softmax(logits, -1)
    rw, ri = torch.topk(ref_p, K, -1)
    assert torch.equal(idx.long(), ri)
    assert torch.allclose(w, rw / rw.sum(-1, keepdim=True), rtol=1e-4, atol=1e-6)
    assert torch.allclose(probs, ref_p, rtol=1e-4, atol=1e-7)
    assert torch.equal(counts.long(), torch.bincount(ri.reshape(-1), minlength=E))
    assert torch.allclose(psum, ref_p.sum(0), rtol=1e-3)
    assert abs(lse.item() - torch.logsumexp(logits, -1).pow(2).sum().item()) < 1e-2 * lse.item()


@pytest.mark.parametrize("E,K,renorm,z", [(128, 8, True, 0.0), (16, 4, False, 1e-3), (60, 2, True, 1e-3), (256, 8, True, 0.0)])
def test_moe_router_backward_kernel(ext, E, K, renorm, z):
    """The fused router-backward kernel against the same formulas written with PyTorch ops in fp32."""
    torch.manual_seed(E + K)
    N, aux_coef = 777, 1e-2
    logits = (torch.randn(N, E, device=DEV) * 2).contiguous()
    probs = torch.softmax(logits, -1)
    ti = torch.topk(probs, K, -1).indices.to(torch.int32).contiguous()
    g = torch.randn(N, K, device=DEV)
    counts = torch.bincount(ti.reshape(-1).long(), minlength=E).to(torch.int32)
    da = torch.tensor([0.37], device=DEV)
    dl = ext.moe_router_bwd(logits, ti, g, counts, da, renorm, aux_coef, z)
    til = ti.long()
    sel = probs.gather(1, til)
    if renorm:
        S = sel.sum(-1, keepdim=True)
        d_sel = g / S - (g * sel).sum(-1, keepdim=True) / (S * S)
    else:
        d_sel = g
    d_probs = torch.zeros_like(probs).scatter_add_(1, til, d_sel) + da * aux_coef * E * (counts.float() / N) / N
    ref = probs * (d_probs - (d_probs * probs).sum(-1, keepdim=True))
    ref = ref + da * z * 2 * torch.logsumexp(logits, -1, keepdim=True) / N * probs
    assert _rel_err(dl, ref) < 6e-3, _rel_err(dl, ref)
    # without the auxiliary term and without top-k gradients the pieces are independent
    dl2 = ext.moe_router_bwd(logits, ti, g, None, None, renorm, aux_coef, z)
    ref2 = probs * (torch.zeros_like(probs).scatter_add_(1, til, d_sel) - (torch.zeros_like(probs).scatter_add_(1, til, d_sel) * probs).sum(-1, keepdim=True))
    assert _rel_err(dl2, ref2) < 6e-3
    _check_flag()


def test_moe_permute_grouped_gemm_unpermute(ext):
    torch.manual_seed(0)
    tokens, C, E, K, Nout = 700, 256, 16, 4, 384
    x = torch.randn(tokens, C, device=DEV).bfloat16()
    ti = torch.stack([torch.randperm(E, device=DEV)[:K] for _ in range(tokens)]).to(torch.int32)
    ti[:, 0] = torch.where(ti[:, 0] == 5, (ti[:, 0] + 1) % E, ti[:, 0])  # leave expert 5 under-used
    counts = torch.bincount(ti.reshape(-1).long(), minlength=E).to(torch.int32)
    cap = tokens * K + E * 128
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    cursors = torch.empty(E, dtype=torch.int32, device=DEV)
    err = ext.error_flag_tensor()
    ext.moe_offsets(counts, offsets, cursors, cap, err)
    ref_off = torch.cat([torch.zeros(1, device=DEV), torch.cumsum((counts + 127) // 128 * 128, 0)]).int()
    assert torch.equal(offsets, ref_off)
    row_map = torch.empty(tokens * K, dtype=torch.int32, device=DEV)
    xp = torch.zeros(cap, C, dtype=torch.bfloat16, device=DEV)
    ext.moe_permute(x, ti, offsets, cursors, row_map, xp, 0, E)
    rm = row_map.view(tokens, K).long()
    assert torch.equal(xp[rm.reshape(-1)], x.repeat_interleave(K, 0))
    e_of_row = torch.bucketize(rm, offsets[1:].long(), right=True)
    assert torch.equal(e_of_row, ti.long())
    assert len(torch.unique(rm)) == tokens * K
    # grouped forward
    w = torch.randn(E, Nout, C, device=DEV).bfloat16() * 0.1
    y = torch.zeros(cap, Nout, dtype=torch.bfloat16, device=DEV)
    ext.gemm_grouped(xp, w, y, offsets, 1, False, False, 1.0, None, None, err)
    ref_y = torch.einsum("rc,rnc->rn", x.repeat_interleave(K, 0).float(), w[ti.reshape(-1).long()].float())
    assert _rel_err(y[rm.reshape(-1)], ref_y) < 6e-3
    # grouped dgrad: dy [R, Nout] . W[g]
    dy = torch.zeros(cap, Nout, dtype=torch.bfloat16, device=DEV)
    dy_rows = torch.randn(tokens * K, Nout, device=DEV).bfloat16()
    dy[rm.reshape(-1)] = dy_rows
    dx = torch.zeros(cap, C, dtype=torch.bfloat16, device=DEV)
    ext.gemm_grouped(dy, w, dx, offsets, 1, True, False, 1.0, None, None, err)
    ref_dx = torch.einsum("rn,rnc->rc", dy_rows.float(), w[ti.reshape(-1).long()].float())
    assert _rel_err(dx[rm.reshape(-1)], ref_dx) < 6e-3
    # grouped wgrad: dW[g] = dy_g^T x_g
    dw = torch.zeros(E, Nout, C, dtype=torch.float32, device=DEV)
    ext.gemm_grouped(dy, xp, dw, offsets, 2, True, True, 1.0, None, None, err)
    ref_dw = torch.zeros_like(dw)
    ref_dw.index_add_(0, ti.reshape(-1).long(), torch.einsum("rn,rc->rnc", dy_rows.float(), x.repeat_interleave(K, 0).float()))
    assert _rel_err(dw, ref_dw) < 6e-3
    # weighted combine + backward
    tw = torch.rand(tokens, K, device=DEV)
    out = ext.moe_unpermute(y, tw, row_map, tokens, K)
    ref_out = (y[rm].float() * tw[..., None]).sum(1)
    assert _rel_err(out, ref_out) < 5e-3
    dout = torch.randn(tokens, Nout, device=DEV).bfloat16()
    d_yp, d_tw = ext.moe_unpermute_bwd(dout, y, tw, row_map)
    assert _rel_err(d_yp[rm.reshape(-1)], (dout.float()[:, None] * tw[..., None]).reshape(-1, Nout)) < 5e-3
    assert _rel_err(d_tw, (y[rm].float() * dout.float()[:, None]).sum(-1)) < 5e-3
    _check_flag()


def test_embedding_rejects_out_of_range_token_ids():
    """An invalid token id must not read outside the table: the row is zero-filled and the error flag is raised."""
    from surogate_b200.ops import check_device_errors, ext

    e = ext()
    check_device_errors()
    table = torch.randn(64, 128, device="cuda", dtype=torch.bfloat16)
    tok = torch.tensor([[3, -100, 63, 64]], device="cuda", dtype=torch.int32)
    out = e.embedding_fwd(tok, table)
    assert torch.equal(out[0, 0], table[3]) and torch.equal(out[0, 2], table[63])
    assert out[0, 1].abs().sum() == 0 and out[0, 3].abs().sum() == 0
    with pytest.raises(RuntimeError, match="token id"):
        check_device_errors()
    check_device_errors()  # the flag was reset by the failed check


def test_cross_entropy_row_weights_and_topk_distillation():
    """The CE kernel's per-row weights (DPO / GRPO) and top-K KD term against an fp32 autograd reference."""
    from surogate_b200.ops import ext

    e = ext()
    torch.manual_seed(0)
    rows, V, K = 48, 4096, 16
    logits = (torch.randn(rows, V, device="cuda") * 3).bfloat16()
    tgt = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    tgt[5] = -100
    rw = torch.randn(rows, device="cuda")
    teacher = torch.log_softmax(torch.randn(rows, V, device="cuda") * 2, -1)
    kl, ki = teacher.topk(K, -1)
    scale = torch.tensor([0.5], device="cuda")
    ref = logits.float().clone().requires_grad_(True)
    lp = torch.log_softmax(ref, -1)
    valid = (tgt >= 0).float()
    ce = -lp.gather(1, tgt.clamp_min(0).long()[:, None]).squeeze(1) * valid
    kd = (kl.exp() * (kl - lp.gather(1, ki))).sum(1) * valid
    (0.5 * ((ce * rw).sum() + 0.25 * kd.sum())).backward()
    work = logits.clone()
    kd_out = torch.empty(rows, device="cuda")
    loss = e.cross_entropy_fwd_bwd(work, tgt, scale, 1.0, True, rw, ki.to(torch.int32).contiguous(), kl.contiguous(), 0.25, kd_out)
    torch.testing.assert_close(loss, ce.detach(), rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(kd_out, kd.detach(), rtol=5e-3, atol=5e-3)
    err = (work.float() - ref.grad).abs().max().item()
    assert err < 2e-2 * ref.grad.abs().max().item() + 1e-3, err
    assert work[5].abs().sum() == 0


def test_barrier_wait_runs_out_and_reports_instead_of_hanging():
    """A peer that never arrives: the barrier kernel gives up after its cycle budget, raises the error word and returns; the
    context stays usable.  (Two local signal pads stand in for two ranks; nothing ever writes the absent rank's arrival.)"""
    from surogate_b200.ops import check_device_errors, ext

    e = ext()
    check_device_errors()
    pads = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]
    err = e.error_flag_tensor()
    t0 = time.time()
    e.symm_barrier([p.data_ptr() for p in pads], 0, 1, 0, err, 0.05)   # I am rank 0 of 2; rank 1 never signals
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    with pytest.raises(RuntimeError, match="wait timed out|error flag"):
        check_device_errors()
    x = torch.ones(8, device="cuda")
    assert float((x * 2).sum()) == 16.0  # the context survived
    check_device_errors()


@pytest.mark.parametrize("dtype,K,silu,packed", [(torch.bfloat16, 4, True, False), (torch.float32, 3, False, False), (torch.float32, 4, True, True),
                                                  (torch.bfloat16, 2, False, True)])
def test_causal_conv1d_forward_and_backward(ext, dtype, K, silu, packed):
    """Depth-wise causal convolution kernels against the PyTorch statement in fp32: tiles that need a halo (T > 64), a channel count that
    is not a multiple of the block, packed documents, the activation folded into backward."""
    from surogate_b200.ops.conv1d import causal_conv1d, causal_conv1d_reference

    torch.manual_seed(1)
    B, T, C = 3, 150, 264
    x = torch.randn(B, T, C, device=DEV).to(dtype).requires_grad_(True)
    w = (torch.randn(C, K, device=DEV) * 0.5).requires_grad_(True)
    b = torch.randn(C, device=DEV).requires_grad_(True)
    ids = None
    if packed:
        ids = torch.zeros(B, T, dtype=torch.int32, device=DEV)
        ids[:, 63:] = 1          # boundaries next to and inside tile edges
        ids[:, 64:] = 2
        ids[:, 130:] = 3
    y = causal_conv1d(x, w, b, "silu" if silu else None, ids)
    dy = torch.randn_like(y)
    y.backward(dy)
    got = (y.detach(), x.grad.clone(), w.grad.clone(), b.grad.clone())
    xr, wr, br = x.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    yr = causal_conv1d_reference(xr, wr, br, "silu" if silu else None, ids)
    yr.backward(dy.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    for name, a, r in zip(("y", "dx", "dw", "db"), got, (yr.detach(), xr.grad, wr.grad, br.grad)):
        assert _rel_err(a, r) < tol, (name, _rel_err(a, r))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_runtime_compiled_elementwise_ops(dtype):
    """Kernels compiled at run time (nvcc -> cubin -> driver API) against their PyTorch statements, forward and backward, and through
    the model-family functions that use them."""
    from surogate_b200.ops import jit
    from surogate_b200.runtime import torch_fns

    torch.manual_seed(0)
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    x = torch.randn(3, 1000, 264, device=DEV).to(dtype)
    for op, ref, kw in ((jit.RELU2, jit._relu2_ref, {}), (jit.SOFTCAP, jit._softcap_ref, {"cap": 2.5})):
        a = x.clone().requires_grad_(True)
        b = x.clone().float().requires_grad_(True)
        y, yr = op(a, **kw), ref(b, **kw)
        dy = torch.randn_like(y)
        y.backward(dy)
        yr.backward(dy.float())
        assert _rel_err(y.detach(), yr.detach()) < tol and _rel_err(a.grad, b.grad) < tol, op.name
    g, u = torch.randn(2, 500, 512, device=DEV).to(dtype), torch.randn(2, 500, 512, device=DEV).to(dtype)
    ga, ua = g.clone().requires_grad_(True), u.clone().requires_grad_(True)
    gb, ub = g.clone().float().requires_grad_(True), u.clone().float().requires_grad_(True)
    y, yr = jit.GEGLU_TANH(ga, ua), jit._geglu_ref(gb, ub)
    dy = torch.randn_like(y)
    y.backward(dy)
    yr.backward(dy.float())
    assert _rel_err(y.detach(), yr.detach()) < tol and _rel_err(ga.grad, gb.grad) < tol and _rel_err(ua.grad, ub.grad) < tol
    packed = torch.cat([u, g], -1)            # [up | gate]
    assert _rel_err(torch_fns.geglu(packed), yr.detach()) < tol
    odd = torch.randn(7, 3, device=DEV).to(dtype)      # not a multiple of the vector width: the PyTorch statement answers
    assert torch.equal(torch_fns.relu2(odd), torch.relu(odd) ** 2)

"""The allocation-free RMSNorm-backward entry point, called the way an embedding application would call it:
through its exported C symbol with raw device pointers.

Such callers (pre-sized serving loops, plug-ins in hosts that own the allocator, latency-critical paths) cannot
call cudaMalloc, so the kernel's workspace lives in the library image.  The test checks that the entry point
reproduces the regular (allocating) entry point on two consecutive calls — the second call reuses the
workspace left behind by the first — and that oversized shapes are refused.
This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from surogate_b200.ops import _build, ext

    ext()  # loads libtorch + the extension, building it when needed
    lib = ctypes.CDLL(_build._so_path())
    fn = lib.sg_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.sg_rmsnorm_bwd_noalloc_strerror.restype = ctypes.c_char_p
    lib.sg_rmsnorm_bwd_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib


def _case(rows, C, seed, with_residual):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dy = torch.randn(rows, C, device="cuda", generator=g).bfloat16()
    x = torch.randn(rows, C, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(C, device="cuda", generator=g)).bfloat16()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    d_res = torch.randn(rows, C, device="cuda", generator=g).bfloat16() if with_residual else None
    return dy, x, w, rstd, d_res


def _fp32_reference(dy, x, w, rstd, d_res):
    """RMSNorm backward in plain fp32 PyTorch: y = x * rstd * w."""
    dyf, xf, wf = dy.float(), x.float(), w.float()
    xhat = xf * rstd[:, None]
    dw = (dyf * xhat).sum(0)
    g = dyf * wf
    dx = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
    if d_res is not None:
        dx = dx + d_res.float()
    return dx, dw


def test_noalloc_matches_regular_entry_point_twice():
    from surogate_b200.ops import ext

    lib, e = _lib(), ext()
    stream = torch.cuda.current_stream().cuda_stream
    # calls in a row with different shapes and data: each runs on the leftover workspace of the one before.  The widest shape the
    # workspace takes (C = 8192) and row counts below and above the 160-block cap are included.
    for rows, C, seed, with_res in [(777, 4096, 0, True), (300, 1024, 1, False), (96, 8192, 2, True), (2048, 8192, 3, False)]:
        dy, x, w, rstd, d_res = _case(rows, C, seed, with_res)
        ref_dx, ref_dw = e.rmsnorm_bwd(dy, x, w, rstd, d_res)
        f_dx, f_dw = _fp32_reference(dy, x, w, rstd, d_res)
        dx = torch.empty_like(x)
        dw = torch.empty(C, device="cuda", dtype=torch.float32)
        rc = lib.sg_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), d_res.data_ptr() if with_res else None,
                                        dx.data_ptr(), dw.data_ptr(), rows, C, stream)
        assert rc == 0, lib.sg_rmsnorm_bwd_noalloc_strerror(rc)
        torch.cuda.synchronize()
        # same kernels, same per-row arithmetic: dx is bit-identical; dw differs only by the number of partial sums
        assert torch.equal(dx, ref_dx)
        rel = (dw - ref_dw).norm() / ref_dw.norm()
        assert rel < 1e-4, rel.item()
        # and against the fp32 statement of the op (dx is rounded to bf16 by the kernel)
        assert ((dx.float() - f_dx).norm() / f_dx.norm()).item() < 6e-3
        assert ((dw - f_dw).norm() / f_dw.norm()).item() < 2e-3


def test_noalloc_rejects_oversized_and_bad_arguments():
    lib = _lib()
    dy, x, w, rstd, _ = _case(8, 64, 2, False)
    dx, dw = torch.empty_like(x), torch.empty(64, device="cuda")
    p = [dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dw.data_ptr()]
    assert lib.sg_rmsnorm_bwd_noalloc(*p, 8, 16384, None) == 2  # wider than the built-in workspace
    assert lib.sg_rmsnorm_bwd_noalloc(*p, 8, 60, None) == 1  # C not a multiple of 8
    assert lib.sg_rmsnorm_bwd_noalloc(None, *p[1:], 8, 64, None) == 1
    assert lib.sg_rmsnorm_bwd_noalloc(p[0] + 2, *p[1:], 8, 64, None) == 1  # a pointer that is not 16-byte aligned
    assert b"aligned" in lib.sg_rmsnorm_bwd_noalloc_strerror(1)
    assert b"8192" in lib.sg_rmsnorm_bwd_noalloc_strerror(2)

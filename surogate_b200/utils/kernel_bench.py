"""Kernel micro-benchmarks with roofline fractions: ``python -m surogate_b200.utils.kernel_bench <kernel> [--size small|full]``.

Each case times one hand-written kernel with CUDA events (3 warm-up launches, then ``--iters`` timed launches with an
L2 flush — a write of a 256 MB buffer — between them), computes the algorithmic FLOPs and bytes of the launch and reports
achieved TFLOP/s and GB/s as fractions of the peaks measured on this machine class (``MEASURED_PEAKS.json`` at the
repository root: STREAM-style copy bandwidth and library bf16 GEMM throughput; built-in fallbacks when absent).
``--size small`` keeps every case to a few hundred MB so that a profiler capture of one launch ends quickly.

The peer-memory collectives (reduce-scatter, all-gather + FP8 quantise) are timed on ONE GPU with ``--ranks`` local
buffers standing in for the peers' memory: the kernel code and its memory traffic are the real ones, only the links are
not crossed, so the figure is the kernel's ceiling, not a link measurement.
"""
from __future__ import annotations

import argparse
import json
import math
import os
from typing import Callable, Dict, List, Optional

import torch

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks() -> Dict[str, float]:
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(os.path.dirname(os.path.dirname(here)), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    except Exception:  # noqa: BLE001
        return dict(FALLBACK_PEAKS, source="fallback")


class Timer:
    def __init__(self, iters: int, flush: bool = True):
        self.iters = iters
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None

    def __call__(self, fn: Callable[[], None]) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(self.iters):
            if self.flush_buf is not None:
                self.flush_buf.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / self.iters


def _report(name: str, ms: float, flops: float, nbytes: float, peaks, tensor_scale: float = 1.0, extra: Optional[Dict] = None) -> Dict:
    tf, gbs = flops / ms / 1e9, nbytes / ms / 1e6
    row = {"kernel": name, "ms": round(ms, 4), "tflops": round(tf, 1), "gbs": round(gbs, 1),
           "frac_of_bf16_gemm_peak": round(tf / (peaks["bf16_tflops"] * tensor_scale), 3) if flops else None,
           "frac_of_copy_bandwidth": round(gbs / peaks["hbm_gbs"], 3), "peaks": peaks["source"], **(extra or {})}
    print(json.dumps(row), flush=True)
    return row


# ---------------------------------------------------------------------------------------------- cases
QWEN3_8B_GEMM_SHAPES = [(8192, 6144, 4096), (8192, 4096, 4096), (8192, 24576, 4096), (8192, 4096, 12288), (4096, 151936, 4096), (8192, 8192, 8192)]


def case_gemm(e, t: Timer, peaks, small: bool, dtype: str = "bf16") -> List[Dict]:
    """Own GEMM (automatic tile choice, single-CTA 128x256 tiles, CTA-pair 256x256 tiles) next to the library GEMM of the same
    shape and dtype: ``torch.matmul`` (cuBLAS) for bf16, ``torch._scaled_mm`` (cuBLASLt FP8, per-tensor scales) for FP8.  The
    library calls exist here as comparators only."""
    from ..runtime.ops_cuda import gemm

    shapes = [(4096, 4096, 4096)] if small else QWEN3_8B_GEMM_SHAPES
    if os.environ.get("SUROGATE_BENCH_GEMM_SHAPE"):   # one shape "M,N,K" and only the own kernel: the form a profiler capture wants
        M, N, K = (int(v) for v in os.environ["SUROGATE_BENCH_GEMM_SHAPE"].split(","))
        dt = torch.bfloat16 if dtype == "bf16" else torch.float8_e4m3fn
        a, b = torch.randn(M, K, device="cuda").to(dt), torch.randn(N, K, device="cuda").to(dt)
        d = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        one = torch.ones(1, device="cuda")
        kw = {} if dtype == "bf16" else dict(scale_a=one, scale_b=one)
        tile_n = int(os.environ.get("SUROGATE_BENCH_GEMM_TILE", "0"))
        return [_report(f"gemm_{dtype} {M}x{N}x{K} tile_n={tile_n}", t(lambda: gemm(a, b, d, tile_n=tile_n, **kw)), 2.0 * M * N * K,
                        (M * K + N * K) * a.element_size() + 2 * M * N, peaks, 1.0 if dtype == "bf16" else 2.0)]
    out = []
    for M, N, K in shapes:
        d = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        one = torch.ones(1, device="cuda")
        if dtype == "bf16":
            a, b = torch.randn(M, K, device="cuda").bfloat16(), torch.randn(N, K, device="cuda").bfloat16()
            kw = {}
            lib = lambda: torch.matmul(a, b.t(), out=d)  # noqa: E731
            nb, scale = 2 * (M * K + N * K + M * N), 1.0
        else:
            a, b = torch.randn(M, K, device="cuda").to(torch.float8_e4m3fn), torch.randn(N, K, device="cuda").to(torch.float8_e4m3fn)
            kw = dict(scale_a=one, scale_b=one)
            lib = lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16, out=d)  # noqa: E731
            nb, scale = M * K + N * K + 2 * M * N, 2.0
        fl = 2.0 * M * N * K
        row = _report(f"gemm_{dtype} {M}x{N}x{K}", t(lambda: gemm(a, b, d, **kw)), fl, nb, peaks, scale)
        ms1 = t(lambda: gemm(a, b, d, tile_n=256, **kw))
        ms2 = t(lambda: gemm(a, b, d, tile_n=512, **kw))
        try:
            ms_lib = t(lib)
        except Exception as ex:  # noqa: BLE001
            ms_lib = float("nan")
            row["library_error"] = str(ex)[:120]
        bt = b.t().contiguous()    # [K, N]: the dgrad layout (second operand MN-major)
        at = a.t().contiguous()    # [K, M]: the wgrad layout (both operands MN-major)
        ms_nn = t(lambda: gemm(a, bt, d, b_mn=True, **kw))
        ms_tn = t(lambda: gemm(at, bt, d, a_mn=True, b_mn=True, **kw))
        row.update({"tflops_single_cta": round(fl / ms1 / 1e9, 1), "tflops_cta_pair": round(fl / ms2 / 1e9, 1), "tflops_library": round(fl / ms_lib / 1e9, 1),
                    "ours_over_library": round(ms_lib / row["ms"], 3), "tflops_b_mn": round(fl / ms_nn / 1e9, 1), "tflops_both_mn": round(fl / ms_tn / 1e9, 1)})
        print(json.dumps({"compare": row["kernel"], **{k: row[k] for k in ("tflops", "tflops_single_cta", "tflops_cta_pair", "tflops_library", "ours_over_library",
                                                                          "tflops_b_mn", "tflops_both_mn")}}), flush=True)
        out.append(row)
        del a, b, at, bt, d
    return out


def case_gemm_nvfp4(e, t, peaks, small):
    M, N, K = (4096, 4096, 4096) if small else (8192, 12288, 4096)
    x, w = torch.randn(M, K, device="cuda").bfloat16(), torch.randn(N, K, device="cuda").bfloat16()
    ax, aw = x.abs().max().float().reshape(1), w.abs().max().float().reshape(1)
    qa, sa = e.nvfp4_quantize(x, ax, False, 0, False)[:2]
    qb, sb = e.nvfp4_quantize(w, aw, False, 0, True)[:2]
    d = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    flag = e.error_flag_tensor()
    one = torch.ones(1, device="cuda")
    ms = t(lambda: e.gemm_nvfp4(qa, sa, qb, sb, d, False, 1.0, one, one, flag))
    rows = [_report(f"gemm_nvfp4 {M}x{N}x{K}", ms, 2.0 * M * N * K, (M * K + N * K) * 0.5625 + 2 * M * N, peaks, 4.0)]
    ms = t(lambda: e.nvfp4_quantize(x, ax, False, 0, False))
    rows.append(_report(f"nvfp4_quantize rows {M}x{K}", ms, 0, M * K * 2 + M * K * 0.5625, peaks))
    ms = t(lambda: e.nvfp4_quantize(x, ax, True, 1, False))
    rows.append(_report(f"nvfp4_quantize rows+SR {M}x{K}", ms, 0, M * K * 2 + M * K * 0.5625, peaks))
    ms = t(lambda: e.nvfp4_quantize_transpose(x, ax, True, True, 1, 0x5A5A))
    rows.append(_report(f"nvfp4_quantize_transpose RHT+SR {M}x{K}", ms, 0, M * K * 2 + M * K * 0.5625, peaks))
    return rows


def case_attention(e, t, peaks, small):
    B, T, Hq, Hkv = (1, 2048, 16, 8) if small else (2, 4096, 32, 8)
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * 128, device="cuda").bfloat16()
    sc = 1 / math.sqrt(128)
    out, lse = e.flash_attn_fwd(qkv, Hq, Hkv, sc)
    do = torch.randn_like(out)
    fl = 4.0 * B * Hq * T * T * 128 / 2
    io = qkv.numel() * 2 + out.numel() * 2
    return [_report(f"flash_attn_fwd B{B} T{T} Hq{Hq} Hkv{Hkv}", t(lambda: e.flash_attn_fwd(qkv, Hq, Hkv, sc)), fl, io, peaks),
            _report(f"flash_attn_bwd B{B} T{T} Hq{Hq} Hkv{Hkv}", t(lambda: e.flash_attn_bwd(do, qkv, out, lse, Hq, Hkv, sc)), 2.5 * fl, 2 * io + do.numel() * 2, peaks)]


def case_elementwise(e, t, peaks, small):
    rows, C, M = (8192, 4096, 12288) if not small else (4096, 4096, 4096)
    x = torch.randn(rows, C, device="cuda").bfloat16()
    res = torch.randn_like(x)
    w = torch.ones(C, device="cuda", dtype=torch.bfloat16)
    out = []
    ms = t(lambda: e.rmsnorm_fwd(x, res, w, 1e-6, True, None, None, False))
    out.append(_report(f"rmsnorm_fwd(+residual) {rows}x{C}", ms, 0, 4 * rows * C * 2, peaks))
    _, y, rstd, _ = e.rmsnorm_fwd(x, None, w, 1e-6, True, None, None, False)
    ms = t(lambda: e.rmsnorm_bwd(y, x, w, rstd, res))
    out.append(_report(f"rmsnorm_bwd(+residual grad) {rows}x{C}", ms, 0, 4 * rows * C * 2, peaks))
    u = torch.randn(rows, 2 * M, device="cuda").bfloat16()
    ms = t(lambda: e.swiglu_fwd(u, True, None, None, False))
    out.append(_report(f"swiglu_fwd {rows}x{M}", ms, 0, 3 * rows * M * 2, peaks))
    dy = torch.randn(rows, M, device="cuda").bfloat16()
    ms = t(lambda: e.swiglu_bwd(dy, u))
    out.append(_report(f"swiglu_bwd {rows}x{M}", ms, 0, 5 * rows * M * 2, peaks))
    Hq, Hkv = 32, 8
    qkv = torch.randn(1, rows, (Hq + 2 * Hkv) * 128, device="cuda").bfloat16()
    pos = torch.arange(rows, device="cuda", dtype=torch.int32)[None].contiguous()
    qw = torch.ones(128, device="cuda", dtype=torch.bfloat16)
    ms = t(lambda: e.qk_norm_rope_fwd(qkv, qw, qw, pos, Hq, Hkv, 128, 1e-6, 1e6))
    out.append(_report(f"qk_norm_rope_fwd {rows} tokens Hq{Hq} Hkv{Hkv}", ms, 0, 2 * qkv.numel() * 2, peaks))
    q8 = lambda: e.quantize_fp8(x, torch.ones(1, device="cuda"), torch.zeros(1, device="cuda"), False)  # noqa: E731
    out.append(_report(f"quantize_fp8 {rows}x{C}", t(q8), 0, rows * C * 3, peaks))
    return out


def case_loss(e, t, peaks, small):
    rows, V = (1024, 151936) if small else (4096, 151936)
    logits = torch.randn(rows, V, device="cuda").bfloat16()
    tgt = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    sc = torch.ones(1, device="cuda")
    ms = t(lambda: e.cross_entropy_fwd_bwd(logits, tgt, sc, 1.0, True))
    return [_report(f"cross_entropy_fwd_bwd {rows}x{V}", ms, 0, 3 * rows * V * 2, peaks)]


def case_optimizer(e, t, peaks, small):
    n = (64 << 20) if small else (512 << 20)
    p, g = torch.randn(n, device="cuda").bfloat16(), torch.randn(n, device="cuda").bfloat16()
    m8, v8 = torch.zeros(n, dtype=torch.int8, device="cuda"), torch.zeros(n, dtype=torch.uint8, device="cuda")
    ms_, vs_ = torch.zeros(n // 32, dtype=torch.float16, device="cuda"), torch.zeros(n // 32, dtype=torch.float16, device="cuda")
    mask = torch.ones(n, dtype=torch.uint8, device="cuda")
    hp = torch.tensor([1e-4, 0.9, 0.999, 1e-8, 0.1, 0.1, 0.001, 1.0], device="cuda")
    out = [_report(f"adamw_8bit {n >> 20}M params", t(lambda: e.adamw8_step(p, g, m8, v8, ms_, vs_, mask, hp)), 0, n * (2 + 2 + 2 + 2 + 2 + 1 + 0.25), peaks)]
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    out.append(_report(f"adamw_fp32 {n >> 20}M params", t(lambda: e.adamw_step(p, g, m, v, mask, hp)), 0, n * (2 + 2 + 2 + 16 + 1), peaks))
    out.append(_report(f"sumsq {n >> 20}M bf16", t(lambda: e.sumsq(g)), 0, n * 2, peaks))
    return out


def case_collectives(e, t, peaks, small, ranks: int = 4):
    """Peer-memory kernels with ``ranks`` local buffers standing in for the peers (see the module docstring)."""
    shard = (8 << 20) if small else (32 << 20)
    full = shard * ranks
    bufs = [torch.randn(full, device="cuda").bfloat16() for _ in range(ranks)]
    ptrs = [b.data_ptr() for b in bufs]
    out_s = torch.empty(shard, device="cuda", dtype=torch.bfloat16)
    ss = torch.zeros(1, device="cuda")
    rows = []
    ms = t(lambda: e.reduce_scatter_fused(ptrs, 0, shard, 1, 1.0, out_s, False, ss, 96))
    rows.append(_report(f"reduce_scatter_fused(+scale+sumsq) {ranks} ranks, shard {shard >> 20}M bf16 [local stand-in]", ms, 0, (ranks + 1) * shard * 2, peaks,
                        extra={"link_bytes_if_remote": (ranks - 1) * shard * 2}))
    shards = [torch.randn(shard, device="cuda").bfloat16() for _ in range(ranks)]
    sptr = [s.data_ptr() for s in shards]
    out16 = torch.empty(full, device="cuda", dtype=torch.bfloat16)
    ms = t(lambda: e.all_gather_fused(sptr, 0, shard, 0, full, out16, None, None, 96))
    rows.append(_report(f"all_gather_fused bf16 {ranks} ranks, shard {shard >> 20}M [local stand-in]", ms, 0, 2 * full * 2, peaks,
                        extra={"link_bytes_if_remote": (ranks - 1) * shard * 2}))
    out8 = torch.empty(full, device="cuda", dtype=torch.uint8)
    sc = torch.ones(1, device="cuda")
    ms = t(lambda: e.all_gather_fused(sptr, 0, shard, 0, full, None, out8, sc, 96))
    rows.append(_report(f"all_gather_fused + FP8 quantise {ranks} ranks, shard {shard >> 20}M [local stand-in]", ms, 0, full * 3, peaks,
                        extra={"link_bytes_if_remote": (ranks - 1) * shard * 2}))
    return rows


def case_moe(e, t, peaks, small):
    from ..runtime.ops_cuda import gemm  # noqa: F401

    tokens, E, K, C, M = (4096, 128, 8, 2048, 768)
    if small:
        tokens = 2048
    logits = torch.randn(tokens, E, device="cuda")
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    ps = torch.zeros(E, device="cuda")
    rows = []

    def route():
        counts.zero_()
        return e.moe_softmax_topk(logits, K, True, counts, ps, None, False)

    rows.append(_report(f"moe_softmax_topk {tokens}x{E} top{K}", t(route), 0, tokens * E * 4 + tokens * K * 8, peaks))
    return rows


CASES = {"gemm_bf16": lambda e, t, p, s: case_gemm(e, t, p, s, "bf16"), "gemm_fp8": lambda e, t, p, s: case_gemm(e, t, p, s, "fp8"),
         "gemm_nvfp4": case_gemm_nvfp4, "attention": case_attention, "elementwise": case_elementwise, "loss": case_loss, "optimizer": case_optimizer,
         "collectives": case_collectives, "moe": case_moe}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m surogate_b200.utils.kernel_bench")
    ap.add_argument("kernel", choices=sorted(CASES) + ["all"])
    ap.add_argument("--size", default="full", choices=["small", "full"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args(argv)
    from ..ops import check_device_errors, ext

    e = ext()
    peaks = load_peaks()
    t = Timer(a.iters, flush=not a.no_flush)
    names = sorted(CASES) if a.kernel == "all" else [a.kernel]
    for n in names:
        CASES[n](e, t, peaks, a.size == "small")
    check_device_errors()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

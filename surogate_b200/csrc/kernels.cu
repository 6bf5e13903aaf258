// Memory-bound training kernels for sm_100a: RMSNorm (+residual, +FP8 output) fwd/bwd, QK-norm + RoPE
// fwd/bwd on packed QKV, SwiGLU fwd/bwd (+FP8 output), embedding fwd/bwd, softmax cross-entropy fwd+bwd in
// place, FP8 quantise / abs-max, sum of squares, AdamW (fp32 state and 8-bit state).
// All loads/stores are 16-byte vectors; reductions are warp shuffles + one shared-memory hop.
//
// Replaces csrc/src/kernels/{rmsnorm,qk_norm,rope,swiglu,encoder,fused_classifier,global_norm}.cu,
// recipes/fp8_hybrid/kernels/quant.cu and runtime/optimizers/{adamw,flash_adamw_8bit}.cu of the reference.
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace sg {

using bf16 = __nv_bfloat16;
using bf162 = __nv_bfloat162;

struct alignas(16) Vec8 { bf162 v[4]; };

__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
    const Vec8 t = *reinterpret_cast<const Vec8*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 x = __bfloat1622float2(t.v[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
}
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
    const bf162* t = reinterpret_cast<const bf162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 x = __bfloat1622float2(t[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
}
__device__ __forceinline__ void store8(bf16* p, const float (&f)[8]) {
    Vec8 t;
#pragma unroll
    for (int i = 0; i < 4; ++i) t.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<Vec8*>(p) = t;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
template <bool IS_MAX> __device__ __forceinline__ float block_reduce(float v, float* sh) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    v = (lane < nw) ? sh[lane] : (IS_MAX ? -INFINITY : 0.f);
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    return v;
}
__device__ __forceinline__ void atomic_max_pos(float* addr, float v) {
    if (v > 0.f) atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}
template <bool E5M2> __device__ __forceinline__ uint8_t to_fp8(float v) {
    return E5M2 ? __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2) : __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// ------------------------------------------------------------------------------------------ RMSNorm forward
// one CTA per row.  res_out = residual + x (optional) ; y = res_out * rstd * w ; optionally y also as FP8.
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ residual, const bf16* __restrict__ w,
                                                          bf16* __restrict__ res_out, bf16* __restrict__ y, float* __restrict__ rstd_out,
                                                          uint8_t* __restrict__ y_fp8, const float* __restrict__ fp8_scale, float* __restrict__ amax_out,
                                                          int C, float eps) {
    __shared__ float sh[32];
    const size_t row = blockIdx.x;
    const bf16* xr = x + row * C;
    const bf16* rr = residual ? residual + row * C : nullptr;
    bf16* ro = res_out ? res_out + row * C : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x * 8; c < C; c += blockDim.x * 8) {
        float a[8];
        load8(xr + c, a);
        if (rr) {
            float b[8];
            load8(rr + c, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] += b[i];
            // round to the stored precision so forward and backward see the same residual stream
            store8(ro + c, a);
            load8(ro + c, a);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += a[i] * a[i];
    }
    ss = block_reduce<false>(ss, sh);
    const float rstd = rsqrtf(ss / C + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
    const bf16* src = rr ? ro : xr;
    const float qs = fp8_scale ? __ldg(fp8_scale) : 1.f;
    float amax = 0.f;
    for (int c = threadIdx.x * 8; c < C; c += blockDim.x * 8) {
        float a[8], g[8];
        load8(src + c, a);
        load8(w + c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) { a[i] = a[i] * rstd * g[i]; amax = fmaxf(amax, fabsf(a[i])); }
        if (y) store8(y + row * C + c, a);
        if (y_fp8) {
            uint2 o;
            uint8_t* ob = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
            for (int i = 0; i < 8; ++i) ob[i] = to_fp8<false>(a[i] * qs);
            *reinterpret_cast<uint2*>(y_fp8 + row * C + c) = o;
        }
    }
    if (amax_out) {
        amax = block_reduce<true>(amax, sh);
        if (threadIdx.x == 0) atomic_max_pos(amax_out, amax);
    }
}

// ------------------------------------------------------------------------------------------ RMSNorm backward
// Persistent CTAs stride over rows; each thread owns fixed columns and keeps dw partial sums in registers.
// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ d_res) ; dw_partial[block, C] reduced by a second kernel.
// ITERS = 8-element vectors per thread (C <= blockDim * 8 * ITERS).  The block size follows C (128 threads up to C = 1024, else
// 256) so that no thread idles on narrow rows, and the number of CTAs follows the register budget: narrow rows run many small
// CTAs per SM, which is what hides the two dependent passes (dot product, then dx) of each row.  With ITERS <= 2 the row stays in
// registers between the passes instead of being read again.
constexpr int RB_THREADS = 256;
template <int ITERS>
__global__ void __launch_bounds__(RB_THREADS) rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                                 const float* __restrict__ rstd, const bf16* __restrict__ d_res,
                                                                 bf16* __restrict__ dx, float* __restrict__ dw_partial, int rows, int C) {
    constexpr bool KEEP = ITERS <= 2;
    __shared__ float sh[32];
    float dw[ITERS][8];
    float ww[ITERS][8];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) { dw[it][i] = 0.f; ww[it][i] = 0.f; }
        if (c < C) load8(w + c, ww[it]);
    }
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = static_cast<size_t>(row) * C;
        const float rs = rstd[row];
        float dot = 0.f;
        // the row stays in registers as packed bf16 between the two passes (KEEP), and the incoming residual gradient is requested
        // together with dy and x, so that its latency hides behind the block reduction instead of following it
        uint4 gk[KEEP ? ITERS : 1], ak[KEEP ? ITERS : 1], rk[KEEP ? ITERS : 1];
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int c = (it * blockDim.x + threadIdx.x) * 8;
            if (c < C) {
                const uint4 graw = *reinterpret_cast<const uint4*>(dy + base + c);
                const uint4 araw = *reinterpret_cast<const uint4*>(x + base + c);
                if (KEEP) {
                    gk[it] = graw;
                    ak[it] = araw;
                    if (d_res) rk[it] = *reinterpret_cast<const uint4*>(d_res + base + c);
                }
                float g[8], a[8];
                unpack8(graw, g);
                unpack8(araw, a);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float xhat = a[i] * rs;
                    dot += g[i] * ww[it][i] * xhat;
                    dw[it][i] += g[i] * xhat;
                }
            }
        }
        dot = block_reduce<false>(dot, sh) / C;
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int c = (it * blockDim.x + threadIdx.x) * 8;
            if (c < C) {
                float g[8], a[8], o[8];
                if (KEEP) {
                    unpack8(gk[it], g);
                    unpack8(ak[it], a);
                } else {
                    load8(dy + base + c, g);
                    load8(x + base + c, a);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = rs * (g[i] * ww[it][i] - a[i] * rs * dot);
                if (d_res) {
                    float r[8];
                    if (KEEP) unpack8(rk[it], r);
                    else load8(d_res + base + c, r);
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] += r[i];
                }
                store8(dx + base + c, o);
            }
        }
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 8;
        if (c < C) {
            float* o = dw_partial + static_cast<size_t>(blockIdx.x) * C + c;
            *reinterpret_cast<float4*>(o) = make_float4(dw[it][0], dw[it][1], dw[it][2], dw[it][3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(dw[it][4], dw[it][5], dw[it][6], dw[it][7]);
        }
    }
}
// out[c] += sum over a slice of the partial rows (gridDim.y slices; ``out`` is zeroed by the launcher)
__global__ void column_sum_kernel(const float* __restrict__ partial, float* __restrict__ out, int nblocks, int C) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float s = 0.f;
    for (int b = blockIdx.y; b < nblocks; b += gridDim.y) s += partial[static_cast<size_t>(b) * C + c];
    atomicAdd(out + c, s);
}

// ------------------------------------------------------------------------------------------ SwiGLU
// x = [up | gate] per row (2M); y = silu(gate) * up.  Optional FP8 copy of y with scale + abs-max.
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, uint8_t* __restrict__ y_fp8,
                                                         const float* __restrict__ fp8_scale, float* __restrict__ amax_out, size_t rows, int M,
                                                         const int* __restrict__ rows_limit) {
    __shared__ float sh[32];
    // rows_limit (device): only the first *rows_limit rows are in use (expert buffers sized for the worst case); cost follows the use
    if (rows_limit) rows = min(rows, static_cast<size_t>(max(0, __ldg(rows_limit))));
    const float qs = fp8_scale ? __ldg(fp8_scale) : 1.f;
    float amax = 0.f;
    // grid.x x block covers the M / 8 column vectors, grid.y strides over the rows: no index division, and a thread's consecutive
    // trips touch consecutive rows of the same columns
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c < M) {
        for (size_t row = blockIdx.y; row < rows; row += gridDim.y) {
            float up[8], gate[8], o[8];
            load8(x + row * 2 * M + c, up);
            load8(x + row * 2 * M + M + c, gate);
#pragma unroll
            for (int i = 0; i < 8; ++i) { o[i] = gate[i] / (1.f + __expf(-gate[i])) * up[i]; amax = fmaxf(amax, fabsf(o[i])); }
            if (y) store8(y + row * M + c, o);
            if (y_fp8) {
                uint2 q;
                uint8_t* qb = reinterpret_cast<uint8_t*>(&q);
#pragma unroll
                for (int i = 0; i < 8; ++i) qb[i] = to_fp8<false>(o[i] * qs);
                *reinterpret_cast<uint2*>(y_fp8 + row * M + c) = q;
            }
        }
    }
    if (amax_out) {
        amax = block_reduce<true>(amax, sh);
        if (threadIdx.x == 0) atomic_max_pos(amax_out, amax);
    }
}
// dx (bf16) and / or dx_fp8 (E5M2 with the given scale, recording the abs-max of the unscaled values): when the only reader of the
// gradient is an FP8 GEMM, the bf16 tensor is never written and no separate quantise pass reads it back.
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, bf16* __restrict__ dx, size_t rows, int M,
                                                         const int* __restrict__ rows_limit, uint8_t* __restrict__ dx_fp8, const float* __restrict__ fp8_scale,
                                                         float* __restrict__ amax_out) {
    __shared__ float sh[32];
    if (rows_limit) rows = min(rows, static_cast<size_t>(max(0, __ldg(rows_limit))));
    const float qs = fp8_scale ? __ldg(fp8_scale) : 1.f;
    float amax = 0.f;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    for (size_t row = blockIdx.y; c < M && row < rows; row += gridDim.y) {
        float up[8], gate[8], g[8], du[8], dg[8];
        load8(x + row * 2 * M + c, up);
        load8(x + row * 2 * M + M + c, gate);
        load8(dy + row * M + c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float s = 1.f / (1.f + __expf(-gate[i]));
            du[i] = g[i] * gate[i] * s;
            dg[i] = g[i] * up[i] * s * (1.f + gate[i] * (1.f - s));
        }
        if (dx) {
            store8(dx + row * 2 * M + c, du);
            store8(dx + row * 2 * M + M + c, dg);
        }
        if (dx_fp8) {
            uint2 qu, qg;
            uint8_t* bu = reinterpret_cast<uint8_t*>(&qu);
            uint8_t* bg = reinterpret_cast<uint8_t*>(&qg);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                amax = fmaxf(amax, fmaxf(fabsf(du[i]), fabsf(dg[i])));
                bu[i] = to_fp8<true>(du[i] * qs);
                bg[i] = to_fp8<true>(dg[i] * qs);
            }
            *reinterpret_cast<uint2*>(dx_fp8 + row * 2 * M + c) = qu;
            *reinterpret_cast<uint2*>(dx_fp8 + row * 2 * M + M + c) = qg;
        }
    }
    if (amax_out) {
        amax = block_reduce<true>(amax, sh);
        if (threadIdx.x == 0) atomic_max_pos(amax_out, amax);
    }
}

// ------------------------------------------------------------------------------------------ QK-norm + RoPE
// Half a warp per (token, head); head_dim 128: lane s = lane & 15 of the half holds elements [8s, 8s+8) (one 16-byte access), the
// rotary partner (i +/- 64) lives in lane s ^ 8 of the same half.  A warp works on one token at a time and walks all of its heads,
// two at a time (one per half-warp), so the rotation angles (sin / cos of position x frequency) are evaluated once per token.
// Layout per token: [Hq heads | Hkv heads (K) | Hkv heads (V)] x D.  V heads are copied (forward) / passed through (backward).
constexpr int ROPE_PAIRS_IN_FLIGHT = 4;      // head pairs whose loads are issued before the first is used
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
template <bool BACKWARD>
__global__ void __launch_bounds__(256) qk_norm_rope_kernel(const bf16* __restrict__ in, const bf16* __restrict__ qkv_pre, const bf16* __restrict__ qw,
                                                           const bf16* __restrict__ kw, const int* __restrict__ pos, bf16* __restrict__ out,
                                                           float* __restrict__ q_rstd, float* __restrict__ k_rstd, float* __restrict__ dqw,
                                                           float* __restrict__ dkw, size_t tokens, int Hq, int Hkv, float eps, float log2_theta,
                                                           int lim_h, int lim_w) {
    // Multi-axis rotary positions (vision-language models): when lim_h or lim_w is non-zero, ``pos`` holds three rows of
    // ``tokens`` entries (temporal, height, width) and frequency j uses the height row if j % 3 == 1 and j < lim_h, the width
    // row if j % 3 == 2 and j < lim_w, else the temporal row.
    constexpr int D = 128;
    constexpr int U = ROPE_PAIRS_IN_FLIGHT;
    __shared__ float sdw[2][D];
    const bool multi_axis = (lim_h | lim_w) != 0;
    if (BACKWARD) {
        for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) (&sdw[0][0])[i] = 0.f;
        __syncthreads();
    }
    const int H = Hq + 2 * Hkv;
    const int lane = threadIdx.x & 31;
    const int sub = lane & 15, hsel = lane >> 4;
    const size_t warps_total = static_cast<size_t>(gridDim.x) * (blockDim.x >> 5);
    const bool use_norm = qw != nullptr;
    float dw_acc[2][8];      // this lane's 8 elements: [q|k] norm-weight grads
    float inv[8], wq8[8], wk8[8];
    int axis[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        dw_acc[0][i] = 0.f;
        dw_acc[1][i] = 0.f;
        wq8[i] = use_norm ? __bfloat162float(qw[sub * 8 + i]) : 1.f;
        wk8[i] = use_norm ? __bfloat162float(kw[sub * 8 + i]) : 1.f;
        const int j = (sub * 8 + i) & 63;
        inv[i] = exp2f(-log2_theta * (2.f * j) / D);
        const int m3 = j % 3;
        axis[i] = (m3 == 1 && j < lim_h) ? 1 : ((m3 == 2 && j < lim_w) ? 2 : 0);
    }
    const float sign = (sub < 8) ? -1.f : 1.f;  // first half of the head: x1*c - x2*s ; second half: x2*c + x1*s
    for (size_t tok = blockIdx.x * static_cast<size_t>(blockDim.x >> 5) + (threadIdx.x >> 5); tok < tokens; tok += warps_total) {
        const float p = static_cast<float>(pos[tok]);
        float p_h = p, p_w = p;
        if (multi_axis) {
            p_h = static_cast<float>(pos[tokens + tok]);
            p_w = static_cast<float>(pos[2 * tokens + tok]);
        }
        float cs[8], sn[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) sincosf((axis[i] == 1 ? p_h : (axis[i] == 2 ? p_w : p)) * inv[i], &sn[i], &cs[i]);
        const size_t tbase = tok * static_cast<size_t>(H) * D + sub * 8;
        for (int hb = 0; hb < H; hb += 2 * U) {
            // all loads of this batch of head pairs are issued before any of them is used
            uint4 raws[U], pres[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int h = hb + 2 * u + hsel;
                if (h < H) {
                    const size_t off = tbase + static_cast<size_t>(h) * D;
                    raws[u] = *reinterpret_cast<const uint4*>(in + off);
                    if (BACKWARD && use_norm && h < Hq + Hkv) pres[u] = *reinterpret_cast<const uint4*>(qkv_pre + off);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int h = hb + 2 * u + hsel;
                // a half-warp whose head index ran past H still takes part in the shuffles of the other half's head
                const bool live = h < H;
                const bool is_v = h >= Hq + Hkv;
                const bool is_q = h < Hq;
                const size_t off = tbase + static_cast<size_t>(h) * D;
                if (hb + 2 * u >= H) break;           // both halves past the end (uniform over the warp)
                float v[8];
                if (live) unpack8(raws[u], v);
                else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = 0.f;
                }
                if (!BACKWARD) {
                    float rstd = 1.f;
                    if (use_norm) {
                        float ss = 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
                        ss = half_warp_sum(ss);
                        rstd = rsqrtf(ss / D + eps);
                        if (live && !is_v) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) v[i] = v[i] * rstd * (is_q ? wq8[i] : wk8[i]);
                            if (sub == 0) {
                                if (is_q) q_rstd[tok * Hq + h] = rstd;
                                else k_rstd[tok * Hkv + (h - Hq)] = rstd;
                            }
                        }
                    }
                    float o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float partner = __shfl_xor_sync(0xffffffffu, v[i], 8);
                        o[i] = v[i] * cs[i] + sign * partner * sn[i];
                    }
                    if (live) {
                        if (is_v) *reinterpret_cast<uint4*>(out + off) = raws[u];
                        else store8(out + off, o);
                    }
                } else {
                    // v = d(out).  Inverse rotation: g1 = d1*c + d2*s ; g2 = d2*c - d1*s
                    float g[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float partner = __shfl_xor_sync(0xffffffffu, v[i], 8);
                        g[i] = v[i] * cs[i] - sign * partner * sn[i];
                    }
                    if (use_norm) {
                        float xin[8];
                        const bool normed = live && !is_v;
                        if (normed) unpack8(pres[u], xin);
                        else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) xin[i] = 0.f;
                        }
                        const float rstd = normed ? (is_q ? q_rstd[tok * Hq + h] : k_rstd[tok * Hkv + (h - Hq)]) : 0.f;
                        float dot = 0.f, dn[8], xhat[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            xhat[i] = xin[i] * rstd;
                            dn[i] = g[i] * (is_q ? wq8[i] : wk8[i]);
                            dot += dn[i] * xhat[i];
                        }
                        if (normed) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) dw_acc[is_q ? 0 : 1][i] += g[i] * xhat[i];
                        }
                        dot = half_warp_sum(dot) / D;
#pragma unroll
                        for (int i = 0; i < 8; ++i) g[i] = rstd * (dn[i] - xhat[i] * dot);
                    }
                    if (live) {
                        if (is_v) *reinterpret_cast<uint4*>(out + off) = raws[u];
                        else store8(out + off, g);
                    }
                }
            }
        }
    }
    if (BACKWARD && use_norm) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            atomicAdd(&sdw[0][sub * 8 + i], dw_acc[0][i]);
            atomicAdd(&sdw[1][sub * 8 + i], dw_acc[1][i]);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            atomicAdd(dqw + i, sdw[0][i]);
            atomicAdd(dkw + i, sdw[1][i]);
        }
    }
}

// ------------------------------------------------------------------------------------------ embedding
// A token id outside [0, V) writes zeros for that row and raises the error flag instead of reading outside the table.
__global__ void embedding_fwd_kernel(const int* __restrict__ tokens, const bf16* __restrict__ table, bf16* __restrict__ out, size_t n, int C, int V,
                                     int* __restrict__ error_flag) {
    const size_t nvec = n * (C / 8);
    for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < nvec; v += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t t = v / (C / 8);
        const int c = static_cast<int>(v % (C / 8)) * 8;
        const int tok = tokens[t];
        if (tok < 0 || tok >= V) {
            *reinterpret_cast<uint4*>(out + t * C + c) = make_uint4(0, 0, 0, 0);
            if (c == 0 && error_flag) atomicExch(error_flag, 2);
            continue;
        }
        *reinterpret_cast<uint4*>(out + t * C + c) = *reinterpret_cast<const uint4*>(table + static_cast<size_t>(tok) * C + c);
    }
}
template <typename G> __global__ void embedding_bwd_kernel(const int* __restrict__ tokens, const bf16* __restrict__ d_out, G* __restrict__ d_table, size_t n, int C) {
    const size_t npair = n * (C / 2);
    for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < npair; v += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t t = v / (C / 2);
        const int c = static_cast<int>(v % (C / 2)) * 2;
        const bf162 g = *reinterpret_cast<const bf162*>(d_out + t * C + c);
        G* dst = d_table + static_cast<size_t>(tokens[t]) * C + c;
        if constexpr (sizeof(G) == 2) {
            atomicAdd(reinterpret_cast<bf162*>(dst), g);
        } else {
            const float2 f = __bfloat1622float2(g);
            atomicAdd(dst, f.x);
            atomicAdd(dst + 1, f.y);
        }
    }
}

// Deterministic variant: positions are sorted by token id first; CTA i owns the run of equal ids that STARTS at sorted position i
// (other CTAs leave at once), sums the run's rows in fp32 in sorted order and adds the sum to the table row once.  No atomics, so
// the result does not depend on scheduling.  Ids outside [0, V) are skipped.
template <typename G>
__global__ void __launch_bounds__(256) embedding_bwd_sorted_kernel(const int* __restrict__ sorted_ids, const long long* __restrict__ order,
                                                                   const bf16* __restrict__ d_out, G* __restrict__ d_table, int n, int C, int V) {
    const int i = blockIdx.x;
    const int id = sorted_ids[i];
    if (id < 0 || id >= V || (i > 0 && sorted_ids[i - 1] == id)) return;
    int end = i + 1;
    while (end < n && sorted_ids[end] == id) ++end;
    for (int c = threadIdx.x * 2; c < C; c += blockDim.x * 2) {
        float ax = 0.f, ay = 0.f;
        for (int j = i; j < end; ++j) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const bf162*>(d_out + static_cast<size_t>(order[j]) * C + c));
            ax += f.x;
            ay += f.y;
        }
        G* dst = d_table + static_cast<size_t>(id) * C + c;
        if constexpr (sizeof(G) == 2) {
            const float2 o = __bfloat1622float2(*reinterpret_cast<const bf162*>(dst));
            *reinterpret_cast<bf162*>(dst) = __floats2bfloat162_rn(o.x + ax, o.y + ay);
        } else {
            dst[0] += ax;
            dst[1] += ay;
        }
    }
}

// ------------------------------------------------------------------------------------------ cross-entropy (fwd + bwd in place)
// One CTA per row of bf16 logits [rows, V].  loss[row] = lse - logit[target]; logits are overwritten with
// d_logits = (softmax - onehot) * scale * row_weight[row] (scale read from device memory), zero for ignored rows.
// row_weight is the hook for sequence-level objectives whose gradient is a per-token multiple of the log-likelihood gradient
// (DPO: +-beta*sigmoid(-margin) per sequence; GRPO: clipped ratio x advantage per token).
// Optional knowledge distillation on a teacher's top-K log-probabilities: kd_loss[row] = sum_k p_k (log p_k - log q_k) with
// q the student softmax, and d_logits += kd_weight * (S * q - scatter(p)), S = sum_k p_k.  A row with an ignored target
// contributes neither term.
__global__ void __launch_bounds__(1024) cross_entropy_fwd_bwd_kernel(bf16* __restrict__ logits, const int* __restrict__ targets, float* __restrict__ loss,
                                                                     const float* __restrict__ scale_ptr, float scale_host, int V, int ld,
                                                                     int write_grad, const float* __restrict__ row_weight,
                                                                     const int* __restrict__ kd_idx, const float* __restrict__ kd_logp, int kd_k,
                                                                     float kd_weight, float* __restrict__ kd_loss) {
    __shared__ float sh[32];
    __shared__ float kd_sum_p;
    const size_t row = blockIdx.x;
    bf16* lr = logits + row * ld;
    const int tgt = targets[row];
    if (tgt < 0) {
        if (threadIdx.x == 0) {
            loss[row] = 0.f;
            if (kd_loss) kd_loss[row] = 0.f;
        }
        if (write_grad) {
            const uint4 z = make_uint4(0, 0, 0, 0);
            for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) *reinterpret_cast<uint4*>(lr + c) = z;
        }
        return;
    }
    float mx = -INFINITY, sum = 0.f;
    for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
        float a[8];
        load8(lr + c, a);
        float m = a[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) m = fmaxf(m, a[i]);
        if (m > mx) { sum *= __expf(mx - m); mx = m; }
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += __expf(a[i] - mx);
    }
    const float gmax = block_reduce<true>(mx, sh);
    sum *= __expf(mx - gmax);
    const float gsum = block_reduce<false>(sum, sh);
    const float lse = gmax + __logf(gsum);
    if (threadIdx.x == 0) loss[row] = lse - __bfloat162float(lr[tgt]);
    float S = 0.f;
    if (kd_k > 0) {  // the first warp walks the teacher's top-K entries of this row
        if (threadIdx.x < 32) {
            float kl = 0.f, sp = 0.f;
            for (int k = threadIdx.x; k < kd_k; k += 32) {
                const int j = kd_idx[row * kd_k + k];
                if (j < 0 || j >= V) continue;
                const float lp = kd_logp[row * kd_k + k];
                const float pk = __expf(lp);
                kl += pk * (lp - (__bfloat162float(lr[j]) - lse));
                sp += pk;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) { kl += __shfl_xor_sync(0xffffffffu, kl, o); sp += __shfl_xor_sync(0xffffffffu, sp, o); }
            if (threadIdx.x == 0) { kd_sum_p = sp; if (kd_loss) kd_loss[row] = kl; }
        }
        __syncthreads();
        S = kd_sum_p;
    }
    if (!write_grad) return;
    __syncthreads();
    const float scale = scale_host * (scale_ptr ? __ldg(scale_ptr) : 1.f);
    const float w_ce = scale * (row_weight ? row_weight[row] : 1.f);
    const float w_kd = kd_k > 0 ? scale * kd_weight : 0.f;
    const float w_soft = w_ce + w_kd * S;
    for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
        float a[8];
        load8(lr + c, a);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float g = __expf(a[i] - lse) * w_soft;
            if (c + i == tgt) g -= w_ce;
            a[i] = g;
        }
        store8(lr + c, a);
    }
    if (kd_k > 0) {
        __syncthreads();  // every gradient of the row is written; now subtract the teacher mass at its K positions
        for (int k = threadIdx.x; k < kd_k; k += blockDim.x) {
            const int j = kd_idx[row * kd_k + k];
            if (j < 0 || j >= V) continue;
            bool first = true;  // a repeated index is applied once per occurrence by the lowest k only (sequentially below)
            for (int q = 0; q < k; ++q) first = first && kd_idx[row * kd_k + q] != j;
            if (!first) continue;
            float pm = 0.f;
            for (int q = k; q < kd_k; ++q)
                if (kd_idx[row * kd_k + q] == j) pm += __expf(kd_logp[row * kd_k + q]);
            lr[j] = __float2bfloat16(__bfloat162float(lr[j]) - w_kd * pm);
        }
    }
}

// ------------------------------------------------------------------------------------------ FP8 quantise / abs-max / sum of squares
template <bool E5M2>
__global__ void __launch_bounds__(256) quantize_fp8_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, const float* __restrict__ scale,
                                                           float* __restrict__ amax_out, size_t n, const int* __restrict__ rows_limit, int row_len) {
    __shared__ float sh[32];
    const float s = scale ? __ldg(scale) : 1.f;
    float amax = 0.f;
    if (rows_limit) n = min(n, static_cast<size_t>(max(0, __ldg(rows_limit))) * row_len);   // only the leading rows are in use
    const size_t nvec = n / 8;
    for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < nvec; v += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float a[8];
        load8(x + v * 8, a);
        uint2 o;
        uint8_t* ob = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
        for (int i = 0; i < 8; ++i) { amax = fmaxf(amax, fabsf(a[i])); ob[i] = to_fp8<E5M2>(a[i] * s); }
        *reinterpret_cast<uint2*>(q + v * 8) = o;
    }
    if (amax_out) {
        amax = block_reduce<true>(amax, sh);
        if (threadIdx.x == 0) atomic_max_pos(amax_out, amax);
    }
}
__global__ void __launch_bounds__(256) amax_kernel(const bf16* __restrict__ x, float* __restrict__ amax_out, size_t n, const int* __restrict__ rows_limit,
                                                   int row_len) {
    __shared__ float sh[32];
    float amax = 0.f;
    if (rows_limit) n = min(n, static_cast<size_t>(max(0, __ldg(rows_limit))) * row_len);
    const size_t nvec = n / 8;
    for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < nvec; v += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float a[8];
        load8(x + v * 8, a);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(a[i]));
    }
    amax = block_reduce<true>(amax, sh);
    if (threadIdx.x == 0) atomic_max_pos(amax_out, amax);
}
// vectorised sum of squares: 16-byte loads, tail handled by the first threads
template <typename T> __global__ void __launch_bounds__(512) sumsq_kernel(const T* __restrict__ x, float* __restrict__ partial, size_t n) {
    __shared__ float sh[32];
    constexpr int VEC = 16 / sizeof(T);
    float s = 0.f;
    const size_t nvec = n / VEC;
    const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x, stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t v = tid; v < nvec; v += stride) {
        if constexpr (sizeof(T) == 2) {
            float a[8];
            load8(reinterpret_cast<const bf16*>(x) + v * 8, a);
#pragma unroll
            for (int i = 0; i < 8; ++i) s += a[i] * a[i];
        } else {
            const float4 a = *reinterpret_cast<const float4*>(x + v * 4);
            s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    for (size_t i = nvec * VEC + tid; i < n; i += stride) {
        float v;
        if constexpr (sizeof(T) == 2) v = __bfloat162float(x[i]); else v = x[i];
        s += v * v;
    }
    s = block_reduce<false>(s, sh);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;   // fixed grid -> deterministic second stage on the host side tensor
}

// ------------------------------------------------------------------------------------------ AdamW
// hp (device): [lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, grad_scale] so a captured graph can be replayed.
// Every thread owns 8 consecutive elements (n must be a multiple of 8; shards are multiples of 128).
template <typename T> __device__ __forceinline__ void load8_any(const T* p, float (&f)[8]) {
    if constexpr (sizeof(T) == 2) {
        load8(reinterpret_cast<const bf16*>(p), f);
    } else {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
}
template <typename T> __device__ __forceinline__ void store8_any(T* p, const float (&f)[8]) {
    if constexpr (sizeof(T) == 2) {
        store8(reinterpret_cast<bf16*>(p), f);
    } else {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
}

template <typename P, typename G>
__global__ void __launch_bounds__(256) adamw_fp32_kernel(P* __restrict__ p, const G* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                                                         const uint8_t* __restrict__ decay_mask, const float* __restrict__ hp, size_t n) {
    const float lr = hp[0], b1 = hp[1], b2 = hp[2], eps = hp[3], wd = hp[4], bc1 = hp[5], bc2 = hp[6], gs = hp[7];
    if (gs == 0.f) return;   // clip scale 0 = the step's gradient was not finite: weights and moments stay as they are
    const float ibc1 = 1.f / bc1, ibc2 = 1.f / bc2;
    const size_t nvec = n / 8;
    for (size_t vi = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; vi < nvec; vi += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t i = vi * 8;
        float pv[8], gv[8], mv[8], vv[8];
        load8_any(p + i, pv);
        load8_any(g + i, gv);
        load8_any(m + i, mv);
        load8_any(v + i, vv);
        uint2 mk = make_uint2(0, 0);
        if (decay_mask) mk = *reinterpret_cast<const uint2*>(decay_mask + i);
        const uint8_t* mb = reinterpret_cast<const uint8_t*>(&mk);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float gk = gv[k] * gs;
            mv[k] = b1 * mv[k] + (1.f - b1) * gk;
            vv[k] = b2 * vv[k] + (1.f - b2) * gk * gk;
            const float dec = mb[k] ? wd : 0.f;
            pv[k] = pv[k] * (1.f - lr * dec) - lr * (mv[k] * ibc1) / (sqrtf(vv[k] * ibc2) + eps);
        }
        store8_any(m + i, mv);
        store8_any(v + i, vv);
        store8_any(p + i, pv);
    }
}

// 8-bit state: momentum int8 through softsign (2x/(1+|x|) of the group-normalised value), variance uint8 of sqrt(v),
// groups of 32 with fp16 scales.  Four adjacent lanes (8 elements each) form one group; the group abs-max is two shuffles.
// n must be a multiple of 32.  The kernel moves 10.25 bytes per parameter, so the work per element has to stay below about
// 40 issued instructions to be bound by memory and not by instruction issue.  Hence:
//  * element pairs go through the packed fp32 instructions of sm_100 (fma / mul / add .f32x2: two results per issue slot);
//  * momentum codes are decoded through a 256-entry shared-memory table, variance codes by splicing the byte into the
//    mantissa of 2^23 (one byte-permute), and both are re-encoded by adding 1.5 * 2^23, whose low mantissa byte then IS the
//    rounded two's-complement code (no float<->int conversions, which share an issue port with the special-function unit);
//  * square root and the two reciprocals per element use the hardware approximations;
//  * the weight-decay mask is one byte per 128 parameters (BLOCK_MASK) instead of one per parameter.
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(reinterpret_cast<unsigned long long&>(d)) : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(reinterpret_cast<unsigned long long&>(d)) : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return d;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)), "l"(reinterpret_cast<unsigned long long&>(c)));
    return d;
}
__device__ __forceinline__ float sqrt_fast(float x) {
    float y;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_fast(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float2 splat2(float x) { return make_float2(x, x); }
constexpr float kRoundMagic = 12582912.f;   // 1.5 * 2^23: adding it rounds to the nearest integer and leaves it in the low mantissa bits

// 3 resident CTAs per SM keep everything in registers (80); capping them at 64 for a fourth CTA spills 80 bytes and measured the same
template <typename P, typename G, bool BLOCK_MASK>
__global__ void __launch_bounds__(256, 3) adamw_8bit_kernel(P* __restrict__ p, const G* __restrict__ g, int8_t* __restrict__ m8, uint8_t* __restrict__ v8,
                                                            __half* __restrict__ ms, __half* __restrict__ vs, const uint8_t* __restrict__ decay_mask,
                                                            const float* __restrict__ hp, size_t n) {
    // softsign decode table of the momentum code, indexed by code + 128: y = c/127, m = y / (2 - |y|) (times the group scale)
    __shared__ float m_lut[256];
    {
        const float y = static_cast<float>(static_cast<int>(threadIdx.x) - 128) * (1.f / 127.f);
        m_lut[threadIdx.x] = y / (2.f - fabsf(y));
    }
    __syncthreads();
    const float lr = hp[0], b1 = hp[1], b2 = hp[2], eps = hp[3], wd = hp[4], bc1 = hp[5], bc2 = hp[6], gs = hp[7];
    if (gs == 0.f) return;   // skipped update (non-finite gradient norm): nothing is read or written
    const float2 gs2 = splat2(gs), b1_2 = splat2(b1), omb1_2 = splat2(1.f - b1), b2_2 = splat2(b2), rt_omb2 = splat2(sqrtf(1.f - b2)),
                 sib2_2 = splat2(rsqrtf(bc2)), eps_2 = splat2(eps), nstep_2 = splat2(-lr / bc1), one_2 = splat2(1.f), magic_2 = splat2(kRoundMagic),
                 c254_2 = splat2(254.f), nbias_2 = splat2(-8388608.f);
    const float decay_on = 1.f - lr * wd;
    const char* lut_bytes = reinterpret_cast<const char*>(m_lut);
    const size_t nvec = n / 8;
    constexpr int U = 2;  // vectors per thread per trip
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x * U;
    // warp-uniform trip count so the shuffles always see all 32 lanes
    for (size_t base = (blockIdx.x * static_cast<size_t>(blockDim.x) + (threadIdx.x & ~31)) * U; base < nvec; base += stride) {
        float pv[U][8], gv[U][8];
        uint2 mraw[U], vraw[U], mk[U];
        float sm[U], sq[U];
        bool live[U];
        size_t idx[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {   // issue every load of both vectors before any arithmetic
            const size_t vi = base + u * 32 + (threadIdx.x & 31);
            live[u] = vi < nvec;
            idx[u] = vi * 8;
            mk[u] = make_uint2(0x01010101u, 0x01010101u);
            if (live[u]) {
                load8_any(p + idx[u], pv[u]);
                load8_any(g + idx[u], gv[u]);
                mraw[u] = *reinterpret_cast<const uint2*>(m8 + idx[u]);
                vraw[u] = *reinterpret_cast<const uint2*>(v8 + idx[u]);
                sm[u] = __half2float(ms[vi >> 2]);
                sq[u] = __half2float(vs[vi >> 2]);
                if (decay_mask) {
                    if (BLOCK_MASK) { if (!decay_mask[idx[u] >> 7]) mk[u] = make_uint2(0, 0); }
                    else mk[u] = *reinterpret_cast<const uint2*>(decay_mask + idx[u]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float2 mv[4], sv[4];
            float am = 0.f, av = 0.f;
            if (live[u]) {
                const uint32_t mw[2] = {mraw[u].x ^ 0x80808080u, mraw[u].y ^ 0x80808080u};   // two's-complement codes -> table indices
                const uint32_t vw[2] = {vraw[u].x, vraw[u].y};
                const uint8_t* mb = reinterpret_cast<const uint8_t*>(&mk[u]);
                const float2 smu2 = splat2(sm[u]), squ2 = splat2(sq[u] * (1.f / 255.f));
                const float2 dec_vec = splat2(mk[u].x ? decay_on : 1.f);
#pragma unroll
                for (int j = 0; j < 4; ++j) {       // elements 2j and 2j + 1
                    const uint32_t mword = mw[j >> 1], vword = vw[j >> 1];
                    const int b0 = (2 * j) & 3, b1i = b0 + 1;
                    // table lookups: byte b of the word, times 4, as a byte offset into the table
                    const uint32_t o0 = b0 == 0 ? (mword << 2) & 0x3FCu : (mword >> (8 * b0 - 2)) & 0x3FCu;
                    const uint32_t o1 = (mword >> (8 * b1i - 2)) & 0x3FCu;
                    float2 mi = mul2(make_float2(*reinterpret_cast<const float*>(lut_bytes + o0), *reinterpret_cast<const float*>(lut_bytes + o1)), smu2);
                    // variance codes: 0x4B0000cc is the float 2^23 + cc
                    const float2 vcode = make_float2(__uint_as_float(__byte_perm(vword, 0x4B000000u, 0x7440u | b0)),
                                                     __uint_as_float(__byte_perm(vword, 0x4B000000u, 0x7440u | b1i)));
                    const float2 r = mul2(add2(vcode, nbias_2), squ2);
                    float2 vi2 = mul2(r, r);
                    const float2 gk = mul2(make_float2(gv[u][2 * j], gv[u][2 * j + 1]), gs2);
                    mi = fma2(b1_2, mi, mul2(omb1_2, gk));
                    const float2 gc = mul2(gk, rt_omb2);
                    vi2 = fma2(gc, gc, mul2(b2_2, vi2));
                    const float2 sd = make_float2(sqrt_fast(vi2.x), sqrt_fast(vi2.y));     // sqrt(v)
                    const float2 den = fma2(sd, sib2_2, eps_2);
                    const float2 q = mul2(mi, make_float2(rcp_fast(den.x), rcp_fast(den.y)));
                    const float2 dec = BLOCK_MASK ? dec_vec : make_float2(mb[2 * j] ? decay_on : 1.f, mb[2 * j + 1] ? decay_on : 1.f);
                    const float2 pn = fma2(q, nstep_2, mul2(make_float2(pv[u][2 * j], pv[u][2 * j + 1]), dec));
                    pv[u][2 * j] = pn.x;
                    pv[u][2 * j + 1] = pn.y;
                    mv[j] = mi;
                    sv[j] = sd;
                    am = fmaxf(am, fmaxf(fabsf(mi.x), fabsf(mi.y)));
                    av = fmaxf(av, fmaxf(sd.x, sd.y));
                }
                store8_any(p + idx[u], pv[u]);
            }
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
            av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, 1));
            av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, 2));
            if (live[u]) {
                // fp16 scales rounded up, so normalised values stay within [-1, 1] (up to one rounding of the product, which cannot
                // move a code past +-127 / 255)
                const __half hm = __float2half_ru(fmaxf(am, 1e-30f)), hv = __float2half_ru(fmaxf(av, 1e-30f));
                const float fm = fmaxf(__half2float(hm), 6e-8f), fv = fmaxf(__half2float(hv), 6e-8f);
                const float2 im2 = splat2(rcp_fast(fm)), iv2 = splat2(255.f * rcp_fast(fv));
                uint32_t mcode[4], vcode[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 xn = mul2(mv[j], im2);
                    const float2 ax = make_float2(fabsf(xn.x), fabsf(xn.y));
                    const float2 den = add2(ax, one_2);
                    const float2 y = mul2(xn, make_float2(rcp_fast(den.x), rcp_fast(den.y)));
                    const float2 mc = fma2(y, c254_2, magic_2);          // low mantissa byte = round(254 x / (1 + |x|)) in two's complement
                    const float2 vc = fma2(sv[j], iv2, magic_2);         // low mantissa byte = round(255 s / scale)
                    mcode[j] = __byte_perm(__float_as_uint(mc.x), __float_as_uint(mc.y), 0x0040u);
                    vcode[j] = __byte_perm(__float_as_uint(vc.x), __float_as_uint(vc.y), 0x0040u);
                }
                uint2 mo, vo;
                mo.x = __byte_perm(mcode[0], mcode[1], 0x5410u);
                mo.y = __byte_perm(mcode[2], mcode[3], 0x5410u);
                vo.x = __byte_perm(vcode[0], vcode[1], 0x5410u);
                vo.y = __byte_perm(vcode[2], vcode[3], 0x5410u);
                *reinterpret_cast<uint2*>(m8 + idx[u]) = mo;
                *reinterpret_cast<uint2*>(v8 + idx[u]) = vo;
                if ((threadIdx.x & 3) == 0) { ms[idx[u] >> 5] = __float2half(fm); vs[idx[u] >> 5] = __float2half(fv); }
            }
        }
    }
}

// ============================================================================================ launchers
static inline int grid_for(size_t work_items, int threads, int num_sms, int per_sm = 8) {
    size_t g = (work_items + threads - 1) / threads;
    const size_t cap = static_cast<size_t>(num_sms) * per_sm;
    return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

void rmsnorm_fwd(const void* x, const void* residual, const void* w, void* res_out, void* y, float* rstd, void* y_fp8, const float* fp8_scale,
                 float* amax, int rows, int C, float eps, cudaStream_t s) {
    int threads = C / 8;
    threads = threads > 256 ? 256 : (threads < 32 ? 32 : (threads + 31) / 32 * 32);
    rmsnorm_fwd_kernel<<<rows, threads, 0, s>>>((const bf16*)x, (const bf16*)residual, (const bf16*)w, (bf16*)res_out, (bf16*)y, rstd, (uint8_t*)y_fp8,
                                                fp8_scale, amax, C, eps);
}
int rmsnorm_bwd_blocks(int rows, int num_sms) { return rows < num_sms * 2 ? rows : num_sms * 2; }
static int rmsnorm_bwd_threads(int C) { return C <= 1024 ? 128 : RB_THREADS; }
static int rmsnorm_bwd_iters(int C) {
    const int per = rmsnorm_bwd_threads(C) * 8;
    const int n = (C + per - 1) / per;
    return n <= 1 ? 1 : (n <= 2 ? 2 : (n <= 4 ? 4 : 8));
}
// CTAs for a [rows, C] problem: as many per SM as the register budget of the variant allows (see the kernel comment)
int rmsnorm_bwd_blocks_wide(int rows, int C, int num_sms) {
    const int per_sm = C <= 1024 ? 8 : (C <= 4096 ? 3 : 2);
    return rows < num_sms * per_sm ? rows : num_sms * per_sm;
}
void rmsnorm_bwd_n(const void* dy, const void* x, const void* w, const float* rstd, const void* d_res, void* dx, float* dw_partial, float* dw, int rows,
                   int C, int blocks, cudaStream_t s) {
    const int threads = rmsnorm_bwd_threads(C);
#define SG_RB(IT) rmsnorm_bwd_kernel<IT><<<blocks, threads, 0, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)d_res, (bf16*)dx, dw_partial, rows, C)
    switch (rmsnorm_bwd_iters(C)) {
        case 1: SG_RB(1); break;
        case 2: SG_RB(2); break;
        case 4: SG_RB(4); break;
        default: SG_RB(8); break;
    }
#undef SG_RB
    cudaMemsetAsync(dw, 0, static_cast<size_t>(C) * sizeof(float), s);
    const int slices = blocks >= 64 ? 8 : 1;
    column_sum_kernel<<<dim3((C + 255) / 256, slices), 256, 0, s>>>(dw_partial, dw, blocks, C);
}
void rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* d_res, void* dx, float* dw_partial, float* dw, int rows,
                 int C, int num_sms, cudaStream_t s) {
    rmsnorm_bwd_n(dy, x, w, rstd, d_res, dx, dw_partial, dw, rows, C, rmsnorm_bwd_blocks(rows, num_sms), s);
}
// blocks of 256 threads over the M / 8 column vectors; enough row-blocks to give every SM eight resident blocks
static int swiglu_threads(int M) {
    const int t = (M / 8 + 31) / 32 * 32;
    return t < 256 ? t : 256;       // narrow expert projections: no idle warps in the block
}
static dim3 swiglu_grid(size_t rows, int M, int num_sms) {
    const int threads = swiglu_threads(M);
    const unsigned gx = static_cast<unsigned>((M / 8 + threads - 1) / threads);
    size_t gy = (static_cast<size_t>(num_sms) * (2048 / threads) + gx - 1) / gx;
    if (gy > rows) gy = rows;
    if (gy < 1) gy = 1;
    if (gy > 65535) gy = 65535;
    return dim3(gx, static_cast<unsigned>(gy));
}
void swiglu_fwd(const void* x, void* y, void* y_fp8, const float* fp8_scale, float* amax, size_t rows, int M, int num_sms, cudaStream_t s,
                const int* rows_limit) {
    swiglu_fwd_kernel<<<swiglu_grid(rows, M, num_sms), swiglu_threads(M), 0, s>>>((const bf16*)x, (bf16*)y, (uint8_t*)y_fp8, fp8_scale, amax, rows, M, rows_limit);
}
void swiglu_bwd(const void* dy, const void* x, void* dx, size_t rows, int M, int num_sms, cudaStream_t s, const int* rows_limit, void* dx_fp8,
                const float* fp8_scale, float* amax_out) {
    swiglu_bwd_kernel<<<swiglu_grid(rows, M, num_sms), swiglu_threads(M), 0, s>>>((const bf16*)dy, (const bf16*)x, (bf16*)dx, rows, M, rows_limit,
                                                                             (uint8_t*)dx_fp8, fp8_scale, amax_out);
}
// Zero the output matrices of groups that own no rows (their wgrad tiles are never scheduled): out [G, per_group] of `elem` bytes.
__global__ void __launch_bounds__(256) zero_empty_groups_kernel(uint4* __restrict__ out, const int* __restrict__ offsets, size_t vec_per_group) {
    const int g = blockIdx.y;
    if (offsets[g + 1] != offsets[g]) return;
    uint4* dst = out + static_cast<size_t>(g) * vec_per_group;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < vec_per_group; i += static_cast<size_t>(gridDim.x) * blockDim.x)
        dst[i] = make_uint4(0, 0, 0, 0);
}
void zero_empty_groups(void* out, const int* offsets, int groups, size_t bytes_per_group, cudaStream_t s) {
    zero_empty_groups_kernel<<<dim3(32, groups), 256, 0, s>>>((uint4*)out, offsets, bytes_per_group / 16);
}
void qk_norm_rope_fwd(const void* qkv, const void* qw, const void* kw, const int* pos, void* out, float* q_rstd, float* k_rstd, size_t tokens, int Hq,
                      int Hkv, float eps, float theta, int lim_h, int lim_w, int num_sms, cudaStream_t s) {
    qk_norm_rope_kernel<false><<<grid_for(tokens * 32, 256, num_sms, 8), 256, 0, s>>>((const bf16*)qkv, nullptr, (const bf16*)qw, (const bf16*)kw, pos,
                                                                                   (bf16*)out, q_rstd, k_rstd, nullptr, nullptr, tokens, Hq, Hkv, eps,
                                                                                   log2f(theta), lim_h, lim_w);
}
void qk_norm_rope_bwd(const void* d_out, const void* qkv_pre, const void* qw, const void* kw, const int* pos, void* d_qkv, float* q_rstd,
                      float* k_rstd, float* dqw, float* dkw, size_t tokens, int Hq, int Hkv, float eps, float theta, int lim_h, int lim_w, int num_sms,
                      cudaStream_t s) {
    qk_norm_rope_kernel<true><<<grid_for(tokens * 32, 256, num_sms, 4), 256, 0, s>>>((const bf16*)d_out, (const bf16*)qkv_pre, (const bf16*)qw,
                                                                                     (const bf16*)kw, pos, (bf16*)d_qkv, q_rstd, k_rstd, dqw, dkw, tokens,
                                                                                     Hq, Hkv, eps, log2f(theta), lim_h, lim_w);
}
void embedding_fwd(const int* tokens, const void* table, void* out, size_t n, int C, int V, int* error_flag, int num_sms, cudaStream_t s) {
    embedding_fwd_kernel<<<grid_for(n * (C / 8), 256, num_sms), 256, 0, s>>>(tokens, (const bf16*)table, (bf16*)out, n, C, V, error_flag);
}
void embedding_bwd(const int* tokens, const void* d_out, void* d_table, int grad_fp32, size_t n, int C, int num_sms, cudaStream_t s) {
    const int grid = grid_for(n * (C / 2), 256, num_sms);
    if (grad_fp32) embedding_bwd_kernel<float><<<grid, 256, 0, s>>>(tokens, (const bf16*)d_out, (float*)d_table, n, C);
    else embedding_bwd_kernel<bf16><<<grid, 256, 0, s>>>(tokens, (const bf16*)d_out, (bf16*)d_table, n, C);
}
void embedding_bwd_sorted(const int* sorted_ids, const long long* order, const void* d_out, void* d_table, int grad_fp32, int n, int C, int V,
                          cudaStream_t s) {
    if (n <= 0) return;
    if (grad_fp32) embedding_bwd_sorted_kernel<float><<<n, 256, 0, s>>>(sorted_ids, order, (const bf16*)d_out, (float*)d_table, n, C, V);
    else embedding_bwd_sorted_kernel<bf16><<<n, 256, 0, s>>>(sorted_ids, order, (const bf16*)d_out, (bf16*)d_table, n, C, V);
}
void cross_entropy_fwd_bwd(void* logits, const int* targets, float* loss, const float* scale_ptr, float scale_host, int rows, int V, int ld,
                           int write_grad, const float* row_weight, const int* kd_idx, const float* kd_logp, int kd_k, float kd_weight, float* kd_loss,
                           cudaStream_t s) {
    cross_entropy_fwd_bwd_kernel<<<rows, 1024, 0, s>>>((bf16*)logits, targets, loss, scale_ptr, scale_host, V, ld, write_grad, row_weight, kd_idx,
                                                       kd_logp, kd_k, kd_weight, kd_loss);
}
void quantize_fp8(const void* x, void* q, const float* scale, float* amax, size_t n, int e5m2, int num_sms, cudaStream_t s, const int* rows_limit,
                  int row_len) {
    const int grid = grid_for(n / 8, 256, num_sms);
    if (e5m2) quantize_fp8_kernel<true><<<grid, 256, 0, s>>>((const bf16*)x, (uint8_t*)q, scale, amax, n, rows_limit, row_len);
    else quantize_fp8_kernel<false><<<grid, 256, 0, s>>>((const bf16*)x, (uint8_t*)q, scale, amax, n, rows_limit, row_len);
}
void amax_bf16(const void* x, float* amax, size_t n, int num_sms, cudaStream_t s, const int* rows_limit, int row_len) {
    amax_kernel<<<grid_for(n / 8, 256, num_sms), 256, 0, s>>>((const bf16*)x, amax, n, rows_limit, row_len);
}
void sumsq(const void* x, int is_fp32, float* partial, int nblocks, size_t n, cudaStream_t s) {
    if (is_fp32) sumsq_kernel<float><<<nblocks, 512, 0, s>>>((const float*)x, partial, n);
    else sumsq_kernel<bf16><<<nblocks, 512, 0, s>>>((const bf16*)x, partial, n);
}
void adamw_fp32(void* p, int p_fp32, const void* g, int g_fp32, float* m, float* v, const uint8_t* mask, const float* hp, size_t n, int num_sms,
                cudaStream_t s) {
    const int grid = grid_for(n / 8, 256, num_sms);
    if (p_fp32 && g_fp32) adamw_fp32_kernel<float, float><<<grid, 256, 0, s>>>((float*)p, (const float*)g, m, v, mask, hp, n);
    else if (p_fp32) adamw_fp32_kernel<float, bf16><<<grid, 256, 0, s>>>((float*)p, (const bf16*)g, m, v, mask, hp, n);
    else if (g_fp32) adamw_fp32_kernel<bf16, float><<<grid, 256, 0, s>>>((bf16*)p, (const float*)g, m, v, mask, hp, n);
    else adamw_fp32_kernel<bf16, bf16><<<grid, 256, 0, s>>>((bf16*)p, (const bf16*)g, m, v, mask, hp, n);
}
void adamw_8bit(void* p, int p_fp32, const void* g, int g_fp32, void* m8, void* v8, void* ms, void* vs, const uint8_t* mask, int block_mask,
                const float* hp, size_t n, int num_sms, cudaStream_t s) {
    const int grid = grid_for(n / 16, 256, num_sms, 16);
#define SG_A8(PT, GT, BM) adamw_8bit_kernel<PT, GT, BM><<<grid, 256, 0, s>>>((PT*)p, (const GT*)g, (int8_t*)m8, (uint8_t*)v8, (__half*)ms, (__half*)vs, mask, hp, n)
    if (block_mask) {
        if (p_fp32 && g_fp32) SG_A8(float, float, true); else if (p_fp32) SG_A8(float, bf16, true); else if (g_fp32) SG_A8(bf16, float, true); else SG_A8(bf16, bf16, true);
    } else {
        if (p_fp32 && g_fp32) SG_A8(float, float, false); else if (p_fp32) SG_A8(float, bf16, false); else if (g_fp32) SG_A8(bf16, float, false); else SG_A8(bf16, bf16, false);
    }
#undef SG_A8
}

}  // namespace sg

// NVFP4 quantisation for sm_100a: E2M1 values with two-level scaling — one FP8 (UE4M3) scale per 16 elements of
// the contraction dimension and one fp32 scale per tensor.
//
//   global encode  ge = (448 * 6) / amax(tensor)                 (device scalar, from an abs-max pass)
//   block scale    sf = e4m3( amax(block16) * ge / 6 )           (stored; decodes to sfd)
//   element        q  = e2m1( x * ge / sfd )                     (round-to-nearest-even, or stochastic for gradients)
//   decode         x ~= q * sfd / ge        =>  GEMM result is scaled by 1 / (ge_a * ge_b) in its epilogue
//
// Scale factors are written in the 128x4 "atom" layout the tensor core reads through TMEM: for row r and 16-element
// block kb, byte ((r/128)*atoms_k + kb/4)*512 + (r%32)*16 + ((r%128)/32)*4 + kb%4.
//
// Kernels: row-wise quantise (blocks along the contiguous dimension), transpose-quantise (blocks along the row
// dimension of the input, i.e. the quantised transpose; optional 16x16 random Hadamard transform applied along the
// block before quantisation, used for weight-gradient operands), 2-D 16x16 weight blocks (one scale shared by a
// 16x16 tile so W and W^T quantise consistently), and dequantise (tests, bf16 fallback GEMM).
//
// Replaces recipes/nvfp4/kernels/{quant_fp4,quant_nvfp4_cutlass,hadamard}.cu of the reference.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "nvfp4_kernels.h"

namespace sg {

using bf16 = __nv_bfloat16;
using bf162 = __nv_bfloat162;

__device__ __forceinline__ size_t sf_offset(int r, int kb, int atoms_k) {
    return (static_cast<size_t>(r >> 7) * atoms_k + (kb >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (kb & 3);
}

// counter-based hash -> uniform float in [0,1)
__device__ __forceinline__ float hash_uniform(uint32_t seed, uint64_t idx) {
    uint64_t z = idx + 0x9E3779B97F4A7C15ull * (static_cast<uint64_t>(seed) + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return static_cast<float>(static_cast<uint32_t>(z >> 40)) * (1.0f / 16777216.0f);
}

// e2m1 code (4 bits: sign | 3-bit magnitude index into {0, .5, 1, 1.5, 2, 3, 4, 6}), round-to-nearest-even on the grid
__device__ __forceinline__ uint32_t e2m1_rn(float v) {
    const uint32_t sign = v < 0.f ? 8u : 0u;
    const float a = fminf(fabsf(v), 6.f);
    uint32_t code;
    if (a <= 0.25f) code = 0;
    else if (a < 0.75f) code = 1;
    else if (a <= 1.25f) code = 2;
    else if (a < 1.75f) code = 3;
    else if (a <= 2.5f) code = 4;
    else if (a < 3.5f) code = 5;
    else if (a <= 5.0f) code = 6;
    else code = 7;
    return sign | code;
}
__device__ __forceinline__ float e2m1_value(uint32_t code) {
    const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    const float m = mag[code & 7];
    return (code & 8) ? -m : m;
}
// stochastic rounding between the two neighbouring grid points (unbiased for |v| <= 6)
__device__ __forceinline__ uint32_t e2m1_sr(float v, float u) {
    const uint32_t sign = v < 0.f ? 8u : 0u;
    const float a = fminf(fabsf(v), 6.f);
    const float grid[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    int lo = 0;
#pragma unroll
    for (int i = 1; i < 8; ++i)
        if (a >= grid[i]) lo = i;
    if (lo == 7) return sign | 7u;
    const float p = (a - grid[lo]) / (grid[lo + 1] - grid[lo]);
    return sign | static_cast<uint32_t>(u < p ? lo + 1 : lo);
}

__device__ __forceinline__ float decode_e4m3(uint8_t b) {
    __nv_fp8_e4m3 t;
    t.__x = b;
    return static_cast<float>(t);
}

// quantise one block of 16 floats: returns 8 packed bytes in `out` (two uint32) and the scale byte
template <bool SR>
__device__ __forceinline__ uint8_t quant_block16(const float (&v)[16], float ge, float forced_amax, uint32_t seed, uint64_t base_idx, uint32_t (&out)[2]) {
    float amax = forced_amax;
    if (forced_amax < 0.f) {
        amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    }
    const uint8_t sfb = __nv_cvt_float_to_fp8(__fdiv_rn(__fmul_rn(amax, ge), 6.f), __NV_SATFINITE, __NV_E4M3);
    const float sfd = decode_e4m3(sfb);
    const float mul = sfd > 0.f ? ge / sfd : 0.f;
    out[0] = out[1] = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float s = v[i] * mul;
        const uint32_t c = SR ? e2m1_sr(s, hash_uniform(seed, base_idx + i)) : e2m1_rn(s);
        out[i >> 3] |= c << ((i & 7) * 4);   // element 2j in the low nibble of byte j
    }
    return sfb;
}

// Four-over-six (round to nearest only): the block is quantised twice, once with its abs-max mapped to the top grid value 6 and
// once mapped to 4 (the grid {0, .5, 1, 1.5, 2, 3, 4} then has no gap between 4 and 6 to fall into), and the mapping with the smaller
// squared reconstruction error is kept.  `err_group` > 1 shares the decision between that many adjacent lanes (16 for the 16 x 16
// weight tiles, whose rows must agree on one scale).  The tensor encode factor is 1536 (= 256 * 6 = 384 * 4), so that both block
// scales stay inside the UE4M3 range.
__device__ __forceinline__ uint8_t quant_block16_4o6(const float (&v)[16], float ge, float forced_amax, uint32_t (&out)[2], int err_group) {
    float amax = forced_amax;
    if (forced_amax < 0.f) {
        amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    }
    uint8_t sfb[2];
    uint32_t codes[2][2];
    float err[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        sfb[t] = __nv_cvt_float_to_fp8(__fdiv_rn(__fmul_rn(amax, ge), t == 0 ? 6.f : 4.f), __NV_SATFINITE, __NV_E4M3);
        const float sfd = decode_e4m3(sfb[t]);
        const float mul = sfd > 0.f ? ge / sfd : 0.f;
        codes[t][0] = codes[t][1] = 0;
        float e = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float s = v[i] * mul;
            const uint32_t c = e2m1_rn(s);
            const float d = (e2m1_value(c) - s) * sfd;      // error in units of x * ge
            e += d * d;
            codes[t][i >> 3] |= c << ((i & 7) * 4);
        }
        err[t] = e;
    }
    for (int o = err_group >> 1; o > 0; o >>= 1) {
        err[0] += __shfl_xor_sync(0xffffffffu, err[0], o);
        err[1] += __shfl_xor_sync(0xffffffffu, err[1], o);
    }
    const int pick = err[1] < err[0] ? 1 : 0;
    out[0] = codes[pick][0];
    out[1] = codes[pick][1];
    return sfb[pick];
}

__device__ __forceinline__ void load16(const bf16* p, float (&v)[16]) {
    const uint4 a = *reinterpret_cast<const uint4*>(p), b = *reinterpret_cast<const uint4*>(p + 8);
    const bf162* pa = reinterpret_cast<const bf162*>(&a);
    const bf162* pb = reinterpret_cast<const bf162*>(&b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
        v[2 * i] = x.x; v[2 * i + 1] = x.y; v[8 + 2 * i] = y.x; v[8 + 2 * i + 1] = y.y;
    }
}

// in-register 16-point Hadamard with random signs (orthonormal: scaled by 1/4)
__device__ __forceinline__ void hadamard16(float (&v)[16], uint32_t sign_mask) {
#pragma unroll
    for (int i = 0; i < 16; ++i)
        if ((sign_mask >> i) & 1u) v[i] = -v[i];
#pragma unroll
    for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if ((i & h) == 0) {
                const float a = v[i], b = v[i + h];
                v[i] = a + b;
                v[i + h] = a - b;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] *= 0.25f;
}

// ------------------------------------------------------------------------------------------ row-wise quantise
// x [rows, K] bf16 (K % 16 == 0) -> q [rows, K/2] bytes, sf in atom layout.  block2d: scales are shared by 16x16 tiles (rows % 16 == 0).
template <bool SR>
__global__ void __launch_bounds__(256) nvfp4_quantize_rows_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                                  const float* __restrict__ amax_tensor, int rows, int K, int atoms_k, uint32_t seed,
                                                                  int block2d, int four_over_six) {
    const float at = __ldg(amax_tensor);
    const float ge = at > 0.f ? __fdiv_rn(four_over_six ? 1536.f : 2688.f, at) : 1.f;
    const int kblocks = K / 16;
    const size_t total = static_cast<size_t>(rows) * kblocks;
    // warp-uniform trip count: the 16x16-tile path shuffles across lanes
    for (size_t base = blockIdx.x * static_cast<size_t>(blockDim.x) + (threadIdx.x & ~31); base < total; base += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t b = base + (threadIdx.x & 31);
        const bool live = b < total;   // total is a multiple of 16 in the tile path, so 16-lane groups are all-live or all-dead
        int r = 0, kb = 0;
        if (!live) {
        } else if (block2d) {   // consecutive threads walk down the 16 rows of a tile so the tile abs-max is a 16-lane shuffle
            const size_t tile = b >> 4;
            const int tiles_k = kblocks;
            r = static_cast<int>(tile / tiles_k) * 16 + static_cast<int>(b & 15);
            kb = static_cast<int>(tile % tiles_k);
        } else {
            r = static_cast<int>(b / kblocks);
            kb = static_cast<int>(b % kblocks);
        }
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
        if (live) load16(x + static_cast<size_t>(r) * K + kb * 16, v);
        float forced = -1.f;
        if (block2d) {
            float m = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            forced = m;
        }
        uint32_t out[2];
        uint8_t sfb;
        if (!SR && four_over_six) {
            sfb = quant_block16_4o6(v, ge, forced, out, block2d ? 16 : 1);   // before the `live` test: the tile decision is a lane shuffle
            if (!live) continue;
        } else {
            if (!live) continue;
            sfb = quant_block16<SR>(v, ge, forced, seed, static_cast<uint64_t>(r) * K + kb * 16, out);
        }
        *reinterpret_cast<uint2*>(q + static_cast<size_t>(r) * (K / 2) + kb * 8) = make_uint2(out[0], out[1]);
        sf[sf_offset(r, kb, atoms_k)] = sfb;
    }
}

// ------------------------------------------------------------------------------------------ transpose-quantise
// x [R, C] bf16 -> quantised x^T: q [C, R/2], sf for (row = c, block = r/16).  R % 64 == 0, C % 64 == 0.
template <bool SR, bool RHT>
__global__ void __launch_bounds__(256) nvfp4_quantize_transpose_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                                       const float* __restrict__ amax_tensor, int R, int C, int atoms_k, uint32_t seed,
                                                                       uint32_t sign_mask, int four_over_six) {
    __shared__ float tile[64][65];
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    for (int i = threadIdx.x; i < 64 * 8; i += blockDim.x) {   // 64 rows x 8 vectors of 8
        const int rr = i >> 3, cv = (i & 7) * 8;
        const uint4 raw = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r0 + rr) * C + c0 + cv);
        const bf162* p = reinterpret_cast<const bf162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(p[j]);
            tile[rr][cv + 2 * j] = f.x;
            tile[rr][cv + 2 * j + 1] = f.y;
        }
    }
    __syncthreads();
    const float at = __ldg(amax_tensor);
    // the Hadamard transform is orthonormal, so the tensor abs-max bound grows by at most 4x; keep head-room for it
    const float enc = (!SR && four_over_six) ? 1536.f : 2688.f;
    const float ge = at > 0.f ? (RHT ? enc / (at * 2.f) : enc / at) : 1.f;
    const int c = threadIdx.x & 63, rb = threadIdx.x >> 6;   // column, 16-row block within the tile
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = tile[rb * 16 + i][c];
    if (RHT) hadamard16(v, sign_mask);
    uint32_t out[2];
    const int kb = (r0 >> 4) + rb;
    const uint8_t sfb = (!SR && four_over_six) ? quant_block16_4o6(v, ge, -1.f, out, 1)
                                                : quant_block16<SR>(v, ge, -1.f, seed, static_cast<uint64_t>(c0 + c) * R + r0 + rb * 16, out);
    *reinterpret_cast<uint2*>(q + static_cast<size_t>(c0 + c) * (R / 2) + (r0 + rb * 16) / 2) = make_uint2(out[0], out[1]);
    sf[sf_offset(c0 + c, kb, atoms_k)] = sfb;
}

// ------------------------------------------------------------------------------------------ dequantise
__global__ void __launch_bounds__(256) nvfp4_dequantize_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf,
                                                               const float* __restrict__ amax_tensor, float amax_div, bf16* __restrict__ out, int rows,
                                                               int K, int atoms_k, float encode) {
    const float at = __ldg(amax_tensor);
    const float inv_ge = at > 0.f ? at * amax_div / encode : 1.f;
    const int kblocks = K / 16;
    const size_t total = static_cast<size_t>(rows) * kblocks;
    for (size_t b = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; b < total; b += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(b / kblocks), kb = static_cast<int>(b % kblocks);
        const uint2 raw = *reinterpret_cast<const uint2*>(q + static_cast<size_t>(r) * (K / 2) + kb * 8);
        const float s = decode_e4m3(sf[sf_offset(r, kb, atoms_k)]) * inv_ge;
        const uint32_t w[2] = {raw.x, raw.y};
        bf16 o[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = __float2bfloat16_rn(e2m1_value((w[i >> 3] >> ((i & 7) * 4)) & 15u) * s);
        *reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * K + kb * 16) = *reinterpret_cast<const uint4*>(&o[0]);
        *reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * K + kb * 16 + 8) = *reinterpret_cast<const uint4*>(&o[8]);
    }
}

// ============================================================================================ launchers
static int q_grid(size_t items, int num_sms) {
    size_t g = (items + 255) / 256;
    const size_t cap = static_cast<size_t>(num_sms) * 8;
    return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}
void nvfp4_quantize_rows(const void* x, void* q, void* sf, const float* amax_tensor, int rows, int K, int stochastic, uint32_t seed, int block2d,
                         int num_sms, cudaStream_t s, int four_over_six) {
    const int atoms_k = (K / 16 + 3) / 4;
    const int grid = q_grid(static_cast<size_t>(rows) * (K / 16), num_sms);
    if (stochastic) nvfp4_quantize_rows_kernel<true><<<grid, 256, 0, s>>>((const bf16*)x, (uint8_t*)q, (uint8_t*)sf, amax_tensor, rows, K, atoms_k, seed, block2d, 0);
    else nvfp4_quantize_rows_kernel<false><<<grid, 256, 0, s>>>((const bf16*)x, (uint8_t*)q, (uint8_t*)sf, amax_tensor, rows, K, atoms_k, seed, block2d, four_over_six);
}
void nvfp4_quantize_transpose(const void* x, void* q, void* sf, const float* amax_tensor, int R, int C, int stochastic, int hadamard, uint32_t seed,
                              uint32_t sign_mask, cudaStream_t s, int four_over_six) {
    const int atoms_k = (R / 16 + 3) / 4;
    const dim3 grid(C / 64, R / 64);
    const bf16* xp = (const bf16*)x;
    uint8_t* qp = (uint8_t*)q;
    uint8_t* sp = (uint8_t*)sf;
    if (stochastic && hadamard) nvfp4_quantize_transpose_kernel<true, true><<<grid, 256, 0, s>>>(xp, qp, sp, amax_tensor, R, C, atoms_k, seed, sign_mask, four_over_six);
    else if (stochastic) nvfp4_quantize_transpose_kernel<true, false><<<grid, 256, 0, s>>>(xp, qp, sp, amax_tensor, R, C, atoms_k, seed, sign_mask, four_over_six);
    else if (hadamard) nvfp4_quantize_transpose_kernel<false, true><<<grid, 256, 0, s>>>(xp, qp, sp, amax_tensor, R, C, atoms_k, seed, sign_mask, four_over_six);
    else nvfp4_quantize_transpose_kernel<false, false><<<grid, 256, 0, s>>>(xp, qp, sp, amax_tensor, R, C, atoms_k, seed, sign_mask, four_over_six);
}
void nvfp4_dequantize(const void* q, const void* sf, const float* amax_tensor, float amax_div, void* out, int rows, int K, int num_sms, cudaStream_t s,
                      float encode) {
    const int atoms_k = (K / 16 + 3) / 4;
    nvfp4_dequantize_kernel<<<q_grid(static_cast<size_t>(rows) * (K / 16), num_sms), 256, 0, s>>>((const uint8_t*)q, (const uint8_t*)sf, amax_tensor,
                                                                                                  amax_div, (bf16*)out, rows, K, atoms_k, encode);
}

}  // namespace sg

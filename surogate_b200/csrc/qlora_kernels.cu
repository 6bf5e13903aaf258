// Dequantisers of the block-quantised storage formats that frozen base weights use under QLoRA (see quant/codecs.py for the
// formats and their PyTorch statements, which are the oracles of these kernels):
//   NF4     4-bit NormalFloat codes (two per byte, low nibble first), fp32 abs-max per block of 64, or double-quantised abs-max
//           (int8 codes in blocks of 256 with an fp32 scale per block and one fp32 offset)
//   FP8     E4M3 values with one fp32 scale per block of 64 / 128 / 256
//   NVFP4   E2M1 codes with sign bit, one UE4M3 scale per 16 elements, one fp32 tensor scale
//   MXFP4   E2M1 codes with sign bit, one E8M0 (power of two) scale per 32 elements
// Every thread turns 8 codes into 8 bf16 values (one 16-byte store); the per-layer weights of a QLoRA step are rebuilt by these
// kernels twice per step (forward and backward), so they run at memory speed instead of through a chain of PyTorch ops.
//
// Replaces csrc/src/kernels/bnb_quant.cu, block_quant.cu and mxfp4_dequant.cu of the reference.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "qlora_kernels.h"

namespace sg {

using bf16 = __nv_bfloat16;
using bf162 = __nv_bfloat162;

__constant__ float kNf4Levels[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f, -0.28444138169288635f,
                                     -0.18477343022823334f, -0.09105003625154495f, 0.0f, 0.07958029955625534f, 0.16093020141124725f,
                                     0.24611230194568634f, 0.33791524171829224f, 0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
__constant__ float kE2m1Levels[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

__device__ __forceinline__ void store8bf(bf16* dst, const float (&v)[8]) {
    uint4 o;
    bf162* po = reinterpret_cast<bf162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(dst) = o;
}
__device__ __forceinline__ float e2m1_value(uint32_t code) {
    const float m = kE2m1Levels[code & 7u];
    return (code & 8u) ? -m : m;
}

// absmax of block b: plain fp32, or int8 code * scale of its 256-block + offset
__device__ __forceinline__ float nf4_absmax(const float* absmax, const int8_t* absmax_q, const float* absmax_scale, float offset, size_t b) {
    return absmax ? absmax[b] : static_cast<float>(absmax_q[b]) * absmax_scale[b >> 8] + offset;
}

__global__ void __launch_bounds__(256) dequant_nf4_kernel(const uint32_t* __restrict__ codes, const float* __restrict__ absmax, const int8_t* __restrict__ absmax_q,
                                                          const float* __restrict__ absmax_scale, const float* __restrict__ absmax_offset,
                                                          bf16* __restrict__ out, size_t n, int block) {
    const float offset = absmax_offset ? __ldg(absmax_offset) : 0.f;
    for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < n / 8; v += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t w = codes[v];
        const float s = nf4_absmax(absmax, absmax_q, absmax_scale, offset, (v * 8) / block);
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = kNf4Levels[(w >> (4 * i)) & 15u] * s;
        store8bf(out + v * 8, o);
    }
}

__global__ void __launch_bounds__(256) dequant_fp8_block_kernel(const uint2* __restrict__ q, const float* __restrict__ scale, bf16* __restrict__ out, size_t n,
                                                                int block) {
    for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < n / 8; v += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint2 w = q[v];
        const float s = scale[(v * 8) / block];
        const __nv_fp8_storage_t* b = reinterpret_cast<const __nv_fp8_storage_t*>(&w);
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __half2float(__half(__nv_cvt_fp8_to_halfraw(b[i], __NV_E4M3))) * s;
        store8bf(out + v * 8, o);
    }
}

// sf: one byte per 16 elements (UE4M3, read as E4M3); ge_inv: the tensor's fp32 de-scale
__global__ void __launch_bounds__(256) dequant_nvfp4_kernel(const uint32_t* __restrict__ codes, const uint8_t* __restrict__ sf, const float* __restrict__ ge_inv,
                                                            bf16* __restrict__ out, size_t n) {
    const float g = __ldg(ge_inv);
    for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < n / 8; v += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t w = codes[v];
        const float s = __half2float(__half(__nv_cvt_fp8_to_halfraw(sf[(v * 8) >> 4], __NV_E4M3))) * g;
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = e2m1_value((w >> (4 * i)) & 15u) * s;
        store8bf(out + v * 8, o);
    }
}

// scales: one E8M0 byte per 32 elements (value 2^(byte - 127))
__global__ void __launch_bounds__(256) dequant_mxfp4_kernel(const uint32_t* __restrict__ codes, const uint8_t* __restrict__ scales, bf16* __restrict__ out,
                                                            size_t n) {
    for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < n / 8; v += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t w = codes[v];
        const float s = exp2f(static_cast<float>(scales[(v * 8) >> 5]) - 127.f);
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = e2m1_value((w >> (4 * i)) & 15u) * s;
        store8bf(out + v * 8, o);
    }
}

static int grid_of(size_t vecs, int num_sms) {
    const size_t want = (vecs + 255) / 256;
    const size_t cap = static_cast<size_t>(num_sms) * 16;
    return static_cast<int>(want < cap ? (want ? want : 1) : cap);
}

void dequant_nf4(const void* codes, const float* absmax, const int8_t* absmax_q, const float* absmax_scale, const float* absmax_offset, void* out,
                 size_t n, int block, int num_sms, cudaStream_t s) {
    dequant_nf4_kernel<<<grid_of(n / 8, num_sms), 256, 0, s>>>((const uint32_t*)codes, absmax, absmax_q, absmax_scale, absmax_offset, (bf16*)out, n, block);
}
void dequant_fp8_block(const void* q, const float* scale, void* out, size_t n, int block, int num_sms, cudaStream_t s) {
    dequant_fp8_block_kernel<<<grid_of(n / 8, num_sms), 256, 0, s>>>((const uint2*)q, scale, (bf16*)out, n, block);
}
void dequant_nvfp4(const void* codes, const void* sf, const float* ge_inv, void* out, size_t n, int num_sms, cudaStream_t s) {
    dequant_nvfp4_kernel<<<grid_of(n / 8, num_sms), 256, 0, s>>>((const uint32_t*)codes, (const uint8_t*)sf, ge_inv, (bf16*)out, n);
}
void dequant_mxfp4(const void* codes, const void* scales, void* out, size_t n, int num_sms, cudaStream_t s) {
    dequant_mxfp4_kernel<<<grid_of(n / 8, num_sms), 256, 0, s>>>((const uint32_t*)codes, (const uint8_t*)scales, (bf16*)out, n);
}

}  // namespace sg

// Depth-wise causal 1-D convolution over channels-last activations [B, T, C], kernel width K <= 4: the short convolutions of
// Mamba-2 mixers, gated delta-net layers and LFM2 blocks.  y[b,t,c] = bias[c] + sum_k w[c,k] * x[b, t-K+1+k, c] (zero before the
// start of the row or of the packed document), optionally followed by SiLU.
//
// A thread owns 8 consecutive channels (one 16-byte access for bf16) and walks a tile of time steps, keeping the last K-1 inputs in
// registers, so every input element is read once per tile (plus a K-1 halo) and no transpose to [B, C, T] is needed.  The backward
// kernel is the linear part only (dx, dw, dbias from the gradient of the pre-activation); the caller folds the activation's
// derivative into that gradient.  Weight and bias gradients are reduced per thread over its tile, then added with fp32 atomics.
//
// Reference counterpart: csrc/third_party causal-conv1d (vendored Dao-AILab kernels), used by the Mamba-2 / GDN layers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "conv1d_kernels.h"

namespace sg {

using bf16 = __nv_bfloat16;
using bf162 = __nv_bfloat162;
constexpr int CV_TILE_T = 64;
constexpr int CV_MAXK = 4;

template <typename T> __device__ __forceinline__ void cv_load8(const T* p, float (&f)[8]);
template <> __device__ __forceinline__ void cv_load8<bf16>(const bf16* p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const bf162* t = reinterpret_cast<const bf162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(t[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
}
template <> __device__ __forceinline__ void cv_load8<float>(const float* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <typename T> __device__ __forceinline__ void cv_store8(T* p, const float (&f)[8]);
template <> __device__ __forceinline__ void cv_store8<bf16>(bf16* p, const float (&f)[8]) {
    uint4 raw;
    bf162* t = reinterpret_cast<bf162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) t[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}
template <> __device__ __forceinline__ void cv_store8<float>(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

// grid: (ceil(C/8 / blockDim.x), ceil(T / CV_TILE_T), B)
template <typename T, int K, bool SILU>
__global__ void __launch_bounds__(128) causal_conv1d_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                                                const int* __restrict__ seq_id, T* __restrict__ y, int Tn, int C) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    const int b = blockIdx.z;
    const int t0 = blockIdx.y * CV_TILE_T;
    const int t1 = min(Tn, t0 + CV_TILE_T);
    float wk[K][8], bs[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        bs[i] = bias ? bias[c + i] : 0.f;
#pragma unroll
        for (int k = 0; k < K; ++k) wk[k][i] = w[(c + i) * K + k];
    }
    const size_t row = static_cast<size_t>(b) * Tn;
    // hist[j] = x at time t - (K-1) + j for j < K-1 (the taps before the current one), zero outside the row
    float hist[K][8];
    int hid[K];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
        const int t = t0 - (K - 1) + j;
        hid[j] = -1;
        if (t >= 0) {
            cv_load8<T>(x + (row + t) * C + c, hist[j]);
            hid[j] = seq_id ? seq_id[row + t] : 0;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) hist[j][i] = 0.f;
        }
    }
    for (int t = t0; t < t1; ++t) {
        cv_load8<T>(x + (row + t) * C + c, hist[K - 1]);
        const int id = seq_id ? seq_id[row + t] : 0;
        hid[K - 1] = id;
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = bs[i];
#pragma unroll
        for (int k = 0; k < K; ++k) {
            if (hid[k] == id) {
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] += wk[k][i] * hist[k][i];
            }
        }
        if (SILU) {
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = o[i] / (1.f + __expf(-o[i]));
        }
        cv_store8<T>(y + (row + t) * C + c, o);
#pragma unroll
        for (int j = 0; j < K - 1; ++j) {
            hid[j] = hid[j + 1];
#pragma unroll
            for (int i = 0; i < 8; ++i) hist[j][i] = hist[j + 1][i];
        }
    }
}

// dx[t] = sum_k w[k] * dz[t + K-1-k]  (future gradients, same document);  dw[k] += sum_t dz[t] * x[t-K+1+k];  dbias += sum_t dz[t]
template <typename T, int K>
__global__ void __launch_bounds__(128) causal_conv1d_bwd_kernel(const T* __restrict__ dz, const T* __restrict__ x, const float* __restrict__ w,
                                                                const int* __restrict__ seq_id, T* __restrict__ dx, float* __restrict__ dw,
                                                                float* __restrict__ dbias, int Tn, int C) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    const int b = blockIdx.z;
    const int t0 = blockIdx.y * CV_TILE_T;
    const int t1 = min(Tn, t0 + CV_TILE_T);
    float wk[K][8], dwk[K][8], db[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        db[i] = 0.f;
#pragma unroll
        for (int k = 0; k < K; ++k) { wk[k][i] = w[(c + i) * K + k]; dwk[k][i] = 0.f; }
    }
    const size_t row = static_cast<size_t>(b) * Tn;
    // walk the tile backwards in time: fut[j] = dz at time t + j (j = 0 .. K-1), zero past the end of the row
    float fut[K][8];
    int fid[K];
#pragma unroll
    for (int j = 1; j < K; ++j) {
        const int t = (t1 - 1) + j;
        fid[j] = -1;
        if (t < Tn) {
            cv_load8<T>(dz + (row + t) * C + c, fut[j]);
            fid[j] = seq_id ? seq_id[row + t] : 0;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) fut[j][i] = 0.f;
        }
    }
    for (int t = t1 - 1; t >= t0; --t) {
        cv_load8<T>(dz + (row + t) * C + c, fut[0]);
        const int id = seq_id ? seq_id[row + t] : 0;
        fid[0] = id;
        float xin[8], o[8];
        cv_load8<T>(x + (row + t) * C + c, xin);
#pragma unroll
        for (int i = 0; i < 8; ++i) { o[i] = 0.f; db[i] += fut[0][i]; }
        // x[t] is tap k of output t + (K-1-k)
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int j = K - 1 - k;
            if (fid[j] == id) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    o[i] += wk[k][i] * fut[j][i];
                    dwk[k][i] += fut[j][i] * xin[i];
                }
            }
        }
        cv_store8<T>(dx + (row + t) * C + c, o);
#pragma unroll
        for (int j = K - 1; j > 0; --j) {
            fid[j] = fid[j - 1];
#pragma unroll
            for (int i = 0; i < 8; ++i) fut[j][i] = fut[j - 1][i];
        }
    }
    // outputs of the next tile (t1 .. t1+K-2) also read inputs of this tile: their dw terms were counted above through fut[j >= 1]
    // of the first iterations, because x[t] pairs with dz[t + j] wherever that lies.
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (dbias) atomicAdd(dbias + c + i, db[i]);
#pragma unroll
        for (int k = 0; k < K; ++k) atomicAdd(dw + (c + i) * K + k, dwk[k][i]);
    }
}

template <typename T>
static void launch_fwd(const T* x, const float* w, const float* bias, const int* seq_id, T* y, int B, int Tn, int C, int K, int silu, cudaStream_t s) {
    const int threads = 128;
    dim3 grid((C / 8 + threads - 1) / threads, (Tn + CV_TILE_T - 1) / CV_TILE_T, B);
#define SG_CV(KK)                                                                                                     \
    if (silu) causal_conv1d_fwd_kernel<T, KK, true><<<grid, threads, 0, s>>>(x, w, bias, seq_id, y, Tn, C);             \
    else causal_conv1d_fwd_kernel<T, KK, false><<<grid, threads, 0, s>>>(x, w, bias, seq_id, y, Tn, C)
    switch (K) {
        case 1: SG_CV(1); break;
        case 2: SG_CV(2); break;
        case 3: SG_CV(3); break;
        default: SG_CV(4); break;
    }
#undef SG_CV
}
template <typename T>
static void launch_bwd(const T* dz, const T* x, const float* w, const int* seq_id, T* dx, float* dw, float* dbias, int B, int Tn, int C, int K, cudaStream_t s) {
    const int threads = 128;
    dim3 grid((C / 8 + threads - 1) / threads, (Tn + CV_TILE_T - 1) / CV_TILE_T, B);
    switch (K) {
        case 1: causal_conv1d_bwd_kernel<T, 1><<<grid, threads, 0, s>>>(dz, x, w, seq_id, dx, dw, dbias, Tn, C); break;
        case 2: causal_conv1d_bwd_kernel<T, 2><<<grid, threads, 0, s>>>(dz, x, w, seq_id, dx, dw, dbias, Tn, C); break;
        case 3: causal_conv1d_bwd_kernel<T, 3><<<grid, threads, 0, s>>>(dz, x, w, seq_id, dx, dw, dbias, Tn, C); break;
        default: causal_conv1d_bwd_kernel<T, 4><<<grid, threads, 0, s>>>(dz, x, w, seq_id, dx, dw, dbias, Tn, C); break;
    }
}

void causal_conv1d_fwd(const void* x, const float* w, const float* bias, const int* seq_id, void* y, int is_fp32, int B, int T, int C, int K, int silu,
                       cudaStream_t s) {
    if (B <= 0 || T <= 0 || C <= 0) return;
    if (is_fp32) launch_fwd<float>((const float*)x, w, bias, seq_id, (float*)y, B, T, C, K, silu, s);
    else launch_fwd<bf16>((const bf16*)x, w, bias, seq_id, (bf16*)y, B, T, C, K, silu, s);
}
void causal_conv1d_bwd(const void* dz, const void* x, const float* w, const int* seq_id, void* dx, float* dw, float* dbias, int is_fp32, int B, int T, int C,
                       int K, cudaStream_t s) {
    if (B <= 0 || T <= 0 || C <= 0) return;
    if (is_fp32) launch_bwd<float>((const float*)dz, (const float*)x, w, seq_id, (float*)dx, dw, dbias, B, T, C, K, s);
    else launch_bwd<bf16>((const bf16*)dz, (const bf16*)x, w, seq_id, (bf16*)dx, dw, dbias, B, T, C, K, s);
}

}  // namespace sg

// NorMuon on the device: the element-wise and row-wise parts of the update around the Polar-Express iteration (whose matrix
// products run on the tcgen05 GEMM of gemm_sm100.cu).  Per 2-D parameter W [R, C] with gradient G:
//
//   1. normuon_momentum   M <- mu M + (1 - mu) s G ;  U = (1 - mu) s G + mu M  (Nesterov blend, bf16) ;  sum U^2
//                         (s = the clip scale, read from the device hyper-parameter vector; M is kept in bf16)
//   2. normuon_normalise  X = U / (1.01 ||U||_F + 1e-7)   in place: the iteration's starting point has singular values < 1
//   3. (five iterations   X <- a X + (b A + c A^2) X, A = X X^T, on the GEMM kernel)
//   4. normuon_row_stats  v_r <- beta2 v_r + (1 - beta2) mean_c(X_rc^2) ;  S1 += sum_c X_rc^2 ;  S2 += sum_c X_rc^2 / (sqrt(v_r) + eps)^2
//   5. normuon_apply      u = X_rc / (sqrt(v_r) + eps) * sqrt(S1 / S2)            (neuron-wise normalisation that keeps the update's norm)
//                         W <- W - lr wd W [u W > 0] - lr * 0.2 sqrt(max(R, C)) * lr_scale * u   (cautious weight decay)
//
// Hyper-parameters come from the device vector hp = [lr, beta1, beta2, eps, wd, bc1, bc2, clip]: a zero clip scale skips the update.
// Replaces csrc/src/runtime/optimizers/normuon.cu of the reference.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "normuon_kernels.h"

namespace sg {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float nm_block_sum(float v, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    v = lane < nw ? sh[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename G>
__global__ void __launch_bounds__(256) normuon_momentum_kernel(const G* __restrict__ g, bf16* __restrict__ m, bf16* __restrict__ u, float* __restrict__ sumsq,
                                                               const float* __restrict__ hp, float mu, size_t n) {
    __shared__ float sh[32];
    const float gs = hp[7];
    if (gs == 0.f) return;
    float acc = 0.f;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float gv;
        if constexpr (sizeof(G) == 2) gv = __bfloat162float(g[i]); else gv = g[i];
        gv *= gs;
        const float mv = mu * __bfloat162float(m[i]) + (1.f - mu) * gv;
        const float uv = (1.f - mu) * gv + mu * mv;
        const bf16 ub = __float2bfloat16_rn(uv);
        m[i] = __float2bfloat16_rn(mv);
        u[i] = ub;
        const float uf = __bfloat162float(ub);
        acc += uf * uf;
    }
    acc = nm_block_sum(acc, sh);
    if (threadIdx.x == 0 && acc != 0.f) atomicAdd(sumsq, acc);
}

// 8-bit momentum: int8 codes with one fp16 scale per 128 values (linear, symmetric: value = code / 127 * scale).  A warp owns one
// group (4 values per lane), so the group's new absolute maximum is one warp reduction.  n % 128 == 0.
template <typename G>
__global__ void __launch_bounds__(256) normuon_momentum8_kernel(const G* __restrict__ g, int8_t* __restrict__ m8, __half* __restrict__ ms, bf16* __restrict__ u,
                                                                float* __restrict__ sumsq, const float* __restrict__ hp, float mu, size_t n) {
    __shared__ float sh[32];
    const float gs = hp[7];
    if (gs == 0.f) return;
    float acc = 0.f;
    const int lane = threadIdx.x & 31;
    const size_t groups = n / 128;
    const size_t warps = static_cast<size_t>(gridDim.x) * (blockDim.x >> 5);
    for (size_t grp = blockIdx.x * static_cast<size_t>(blockDim.x >> 5) + (threadIdx.x >> 5); grp < groups; grp += warps) {
        const size_t i = grp * 128 + lane * 4;
        const float scale = __half2float(ms[grp]) * (1.f / 127.f);
        const char4 c = *reinterpret_cast<const char4*>(m8 + i);
        float gv[4];
        if constexpr (sizeof(G) == 2) {
            const uint2 raw = *reinterpret_cast<const uint2*>(g + i);
            const __nv_bfloat162* t = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float2 a = __bfloat1622float2(t[0]), b = __bfloat1622float2(t[1]);
            gv[0] = a.x; gv[1] = a.y; gv[2] = b.x; gv[3] = b.y;
        } else {
            const float4 a = *reinterpret_cast<const float4*>(g + i);
            gv[0] = a.x; gv[1] = a.y; gv[2] = a.z; gv[3] = a.w;
        }
        const float mo[4] = {c.x * scale, c.y * scale, c.z * scale, c.w * scale};
        float mv[4], amax = 0.f;
        uint2 uo;
        __nv_bfloat162* ub = reinterpret_cast<__nv_bfloat162*>(&uo);
        float uv[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float gk = gv[k] * gs;
            mv[k] = mu * mo[k] + (1.f - mu) * gk;
            uv[k] = (1.f - mu) * gk + mu * mv[k];
            amax = fmaxf(amax, fabsf(mv[k]));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const __half hs = __float2half_ru(amax);              // rounded up: no code can exceed 127
        const float inv = amax > 0.f ? 127.f / __half2float(hs) : 0.f;
        char4 co;
        co.x = static_cast<signed char>(__float2int_rn(mv[0] * inv));
        co.y = static_cast<signed char>(__float2int_rn(mv[1] * inv));
        co.z = static_cast<signed char>(__float2int_rn(mv[2] * inv));
        co.w = static_cast<signed char>(__float2int_rn(mv[3] * inv));
        *reinterpret_cast<char4*>(m8 + i) = co;
        if (lane == 0) ms[grp] = hs;
        ub[0] = __floats2bfloat162_rn(uv[0], uv[1]);
        ub[1] = __floats2bfloat162_rn(uv[2], uv[3]);
        *reinterpret_cast<uint2*>(u + i) = uo;
        const float2 r0 = __bfloat1622float2(ub[0]), r1 = __bfloat1622float2(ub[1]);
        acc += r0.x * r0.x + r0.y * r0.y + r1.x * r1.x + r1.y * r1.y;
    }
    acc = nm_block_sum(acc, sh);
    if (threadIdx.x == 0 && acc != 0.f) atomicAdd(sumsq, acc);
}

__global__ void __launch_bounds__(256) normuon_normalise_kernel(bf16* __restrict__ x, const float* __restrict__ sumsq, size_t n) {
    const float inv = 1.f / (sqrtf(__ldg(sumsq)) * 1.01f + 1e-7f);
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x)
        x[i] = __float2bfloat16_rn(__bfloat162float(x[i]) * inv);
}

// one CTA per row; sums[0] += row sum of squares, sums[1] += the same divided by (sqrt(v_r) + eps)^2
__global__ void __launch_bounds__(256) normuon_row_stats_kernel(const bf16* __restrict__ x, float* __restrict__ v, float* __restrict__ sums,
                                                                const float* __restrict__ hp, float beta2, int C) {
    __shared__ float sh[32];
    if (hp[7] == 0.f) return;
    const int r = blockIdx.x;
    float acc = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float f = __bfloat162float(x[static_cast<size_t>(r) * C + c]);
        acc += f * f;
    }
    acc = nm_block_sum(acc, sh);
    if (threadIdx.x == 0) {
        const float vr = beta2 * v[r] + (1.f - beta2) * acc / static_cast<float>(C);
        v[r] = vr;
        const float d = sqrtf(vr) + hp[3];
        atomicAdd(&sums[0], acc);
        atomicAdd(&sums[1], acc / (d * d));
    }
}

template <typename W>
__global__ void __launch_bounds__(256) normuon_apply_kernel(W* __restrict__ w, const bf16* __restrict__ x, const float* __restrict__ v,
                                                            const float* __restrict__ sums, const float* __restrict__ hp, float update_scale, int cautious,
                                                            int C, size_t first, size_t count) {
    // elements [first, first + count) of the row-major matrix (a rank may own only part of a matrix whose rows it helped orthogonalise)
    if (hp[7] == 0.f) return;
    const float lr = hp[0], eps = hp[3], wd = hp[4];
    const float renorm = sums[1] > 0.f ? sqrtf(sums[0] / sums[1]) : 0.f;
    for (size_t k = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; k < count; k += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t i = first + k;
        const int r = static_cast<int>(i / C);
        const float u = __bfloat162float(x[i]) / (sqrtf(v[r]) + eps) * renorm;
        float wv;
        if constexpr (sizeof(W) == 2) wv = __bfloat162float(w[k]); else wv = w[k];
        const float decay = (!cautious || u * wv > 0.f) ? wd * lr * wv : 0.f;
        wv = wv - decay - lr * update_scale * u;
        if constexpr (sizeof(W) == 2) w[k] = __float2bfloat16_rn(wv); else w[k] = wv;
    }
}

static int nm_grid(size_t n, int num_sms) {
    size_t g = (n + 255) / 256;
    const size_t cap = static_cast<size_t>(num_sms) * 8;
    return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

void normuon_momentum(const void* g, int g_fp32, void* m, void* u, float* sumsq, const float* hp, float mu, size_t n, int num_sms, cudaStream_t s) {
    if (g_fp32) normuon_momentum_kernel<float><<<nm_grid(n, num_sms), 256, 0, s>>>((const float*)g, (bf16*)m, (bf16*)u, sumsq, hp, mu, n);
    else normuon_momentum_kernel<bf16><<<nm_grid(n, num_sms), 256, 0, s>>>((const bf16*)g, (bf16*)m, (bf16*)u, sumsq, hp, mu, n);
}
void normuon_momentum8(const void* g, int g_fp32, void* m8, void* ms, void* u, float* sumsq, const float* hp, float mu, size_t n, int num_sms, cudaStream_t s) {
    const size_t warps = n / 128;
    size_t grid = (warps + 7) / 8;
    const size_t cap = static_cast<size_t>(num_sms) * 8;
    grid = grid < 1 ? 1 : (grid > cap ? cap : grid);
    if (g_fp32) normuon_momentum8_kernel<float><<<static_cast<int>(grid), 256, 0, s>>>((const float*)g, (int8_t*)m8, (__half*)ms, (bf16*)u, sumsq, hp, mu, n);
    else normuon_momentum8_kernel<bf16><<<static_cast<int>(grid), 256, 0, s>>>((const bf16*)g, (int8_t*)m8, (__half*)ms, (bf16*)u, sumsq, hp, mu, n);
}
void normuon_normalise(void* x, const float* sumsq, size_t n, int num_sms, cudaStream_t s) {
    normuon_normalise_kernel<<<nm_grid(n, num_sms), 256, 0, s>>>((bf16*)x, sumsq, n);
}
void normuon_row_stats(const void* x, float* v, float* sums, const float* hp, float beta2, int R, int C, cudaStream_t s) {
    normuon_row_stats_kernel<<<R, 256, 0, s>>>((const bf16*)x, v, sums, hp, beta2, C);
}
void normuon_apply(void* w, int w_fp32, const void* x, const float* v, const float* sums, const float* hp, float update_scale, int cautious, int C,
                   size_t first, size_t count, int num_sms, cudaStream_t s) {
    if (count == 0) return;
    if (w_fp32) normuon_apply_kernel<float><<<nm_grid(count, num_sms), 256, 0, s>>>((float*)w, (const bf16*)x, v, sums, hp, update_scale, cautious, C, first, count);
    else normuon_apply_kernel<bf16><<<nm_grid(count, num_sms), 256, 0, s>>>((bf16*)w, (const bf16*)x, v, sums, hp, update_scale, cautious, C, first, count);
}

}  // namespace sg

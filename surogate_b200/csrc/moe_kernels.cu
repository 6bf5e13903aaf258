// Mixture-of-experts routing kernels for sm_100a: softmax + top-k (+ counts and probability sums for the
// auxiliary loss), padded expert offsets (device-side scan), token permutation into expert-sorted padded rows,
// weighted un-permute / combine and their backward kernels.  Everything stays on the device: no expert count is
// ever read back by the host, buffers are sized by a static upper bound and the grouped GEMM reads the offsets.
//
// Replaces csrc/src/kernels/moe/{moe_routing_activation,moe_topk,moe_dispatch_permute,moe_backward_dispatch}.cu of
// the reference (whose offset / index kernels run as <<<1,1>>> and whose host code synchronises per layer).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "moe_kernels.h"

namespace sg {

using bf16 = __nv_bfloat16;
using bf162 = __nv_bfloat162;

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ------------------------------------------------------------------------------------------ softmax + top-k
// One warp per token; E <= 256 (8 values per lane).  Writes normalised top-k weights, indices, and accumulates per-expert
// assignment counts and probability sums (for the load-balancing loss) with one atomic per expert per block.
template <int VPL>
__global__ void __launch_bounds__(256) moe_softmax_topk_kernel(const float* __restrict__ logits, float* __restrict__ topk_w, int* __restrict__ topk_idx,
                                                               float* __restrict__ probs_out, int* __restrict__ counts, float* __restrict__ prob_sum,
                                                               float* __restrict__ lse_sq_sum, int tokens, int E, int K, int renorm) {
    extern __shared__ float sh[];   // [E] probability sums, [E] counts (as int)
    float* sh_p = sh;
    int* sh_c = reinterpret_cast<int*>(sh + E);
    for (int i = threadIdx.x; i < E; i += blockDim.x) { sh_p[i] = 0.f; sh_c[i] = 0; }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    float lse_acc = 0.f;
    for (int tok = blockIdx.x * wpb + (threadIdx.x >> 5); tok < tokens; tok += gridDim.x * wpb) {
        float v[VPL];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int e = i * 32 + lane;
            v[i] = e < E ? logits[static_cast<size_t>(tok) * E + e] : -INFINITY;
            mx = fmaxf(mx, v[i]);
        }
        mx = wmax(mx);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) { v[i] = (i * 32 + lane < E) ? __expf(v[i] - mx) : 0.f; sum += v[i]; }
        sum = wsum(sum);
        const float inv = 1.f / sum;
        if (lane == 0) { const float lse = mx + __logf(sum); lse_acc += lse * lse; }
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            v[i] *= inv;
            const int e = i * 32 + lane;
            if (e < E) {
                atomicAdd(&sh_p[e], v[i]);
                if (probs_out) probs_out[static_cast<size_t>(tok) * E + e] = v[i];
            }
        }
        float sel_sum = 0.f, my_w = 0.f;
        int my_idx = 0;
        for (int k = 0; k < K; ++k) {
            float best = -1.f;
            int bi = 0;
#pragma unroll
            for (int i = 0; i < VPL; ++i)
                if (v[i] > best) { best = v[i]; bi = i * 32 + lane; }
            // warp arg-max; ties resolved towards the lower expert index
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
            }
            if ((bi & 31) == lane) v[bi >> 5] = -2.f;   // remove the winner
            sel_sum += best;
            if (lane == k) { my_w = best; my_idx = bi; }
            if (lane == 0) atomicAdd(&sh_c[bi], 1);
        }
        if (lane < K) {
            topk_w[static_cast<size_t>(tok) * K + lane] = renorm ? my_w / sel_sum : my_w;
            topk_idx[static_cast<size_t>(tok) * K + lane] = my_idx;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        if (sh_c[i]) atomicAdd(&counts[i], sh_c[i]);
        if (sh_p[i] != 0.f) atomicAdd(&prob_sum[i], sh_p[i]);
    }
    if (lse_sq_sum && lane == 0 && lse_acc != 0.f) atomicAdd(lse_sq_sum, lse_acc);
}

// ------------------------------------------------------------------------------------------ router backward
// d_logits [tokens, E] (bf16) from the gradients of the top-k weights and of the auxiliary losses; one warp per token, E <= 256.
//   probs = softmax(logits); sel_k = probs[idx_k]
//   d_sel_k = renorm ? g_k / S - (sum_j g_j sel_j) / S^2 : g_k                      (S = sum_k sel_k)
//   d_probs[e] = sum_k [idx_k == e] d_sel_k + aux_grad * counts[e]                  (aux_grad = d_aux * coef * E / tokens^2)
//   d_logits = probs * (d_probs - <d_probs, probs>) + z_grad * lse * probs          (z_grad = d_aux * z_coef * 2 / tokens)
// d_aux arrives as a device scalar (the loss scale); counts are the forward's per-expert assignment counts.
template <int VPL>
__global__ void __launch_bounds__(256) moe_router_bwd_kernel(const float* __restrict__ logits, const int* __restrict__ topk_idx, const float* __restrict__ d_topk_w,
                                                             const int* __restrict__ counts, const float* __restrict__ d_aux, bf16* __restrict__ d_logits,
                                                             int tokens, int E, int K, int renorm, float aux_coef, float z_coef) {
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const float da = d_aux ? __ldg(d_aux) : 0.f;
    const float aux_grad = da * aux_coef * static_cast<float>(E) / (static_cast<float>(tokens) * static_cast<float>(tokens));
    const float z_grad = da * z_coef * 2.f / static_cast<float>(tokens);
    float cnt[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int e = i * 32 + lane;
        cnt[i] = (e < E && counts) ? static_cast<float>(counts[e]) : 0.f;
    }
    for (int tok = blockIdx.x * wpb + (threadIdx.x >> 5); tok < tokens; tok += gridDim.x * wpb) {
        float p[VPL], dp[VPL];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int e = i * 32 + lane;
            p[i] = e < E ? logits[static_cast<size_t>(tok) * E + e] : -INFINITY;
            mx = fmaxf(mx, p[i]);
        }
        mx = wmax(mx);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) { p[i] = (i * 32 + lane < E) ? __expf(p[i] - mx) : 0.f; sum += p[i]; }
        sum = wsum(sum);
        const float inv = 1.f / sum, lse = mx + __logf(sum);
#pragma unroll
        for (int i = 0; i < VPL; ++i) { p[i] *= inv; dp[i] = aux_grad * cnt[i]; }
        // lane k < K owns the k-th selected expert of the token
        const int my_idx = lane < K ? topk_idx[static_cast<size_t>(tok) * K + lane] : -1;
        const float my_g = (lane < K && d_topk_w) ? d_topk_w[static_cast<size_t>(tok) * K + lane] : 0.f;
        float my_sel = 0.f;
        for (int k = 0; k < K; ++k) {
            const int e = __shfl_sync(0xffffffffu, my_idx, k);
            float v = 0.f;
#pragma unroll
            for (int i = 0; i < VPL; ++i)
                if (i * 32 + lane == e) v = p[i];
            v = wsum(v);                          // probability of the k-th selected expert, in every lane
            if (lane == k) my_sel = v;
        }
        float d_sel = my_g;
        if (renorm) {
            const float S = wsum(my_sel), gs = wsum(my_g * my_sel);
            d_sel = my_g / S - gs / (S * S);
        }
        for (int k = 0; k < K; ++k) {
            const int e = __shfl_sync(0xffffffffu, my_idx, k);
            const float d = __shfl_sync(0xffffffffu, d_sel, k);
#pragma unroll
            for (int i = 0; i < VPL; ++i)
                if (i * 32 + lane == e) dp[i] += d;
        }
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) dot += dp[i] * p[i];
        dot = wsum(dot);
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int e = i * 32 + lane;
            if (e < E) d_logits[static_cast<size_t>(tok) * E + e] = __float2bfloat16(p[i] * (dp[i] - dot) + z_grad * lse * p[i]);
        }
    }
}

// ------------------------------------------------------------------------------------------ padded offsets
// offsets[e] = sum_{j<e} round_up(counts[j], 128); one block, warp-level scan.  Also zeroes the per-expert cursors.
__global__ void __launch_bounds__(256) moe_offsets_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ cursors, int E,
                                                          int capacity_rows, int* __restrict__ error_flag) {
    __shared__ int sh[257];
    const int t = threadIdx.x;
    int v = 0;
    if (t < E) v = (counts[t] + 127) / 128 * 128;
    sh[t] = v;
    __syncthreads();
    for (int o = 1; o < 256; o <<= 1) {   // Hillis-Steele inclusive scan (E <= 256)
        int add = t >= o ? sh[t - o] : 0;
        __syncthreads();
        sh[t] += add;
        __syncthreads();
    }
    if (t < E) { offsets[t + 1] = sh[t]; cursors[t] = 0; }
    if (t == 0) {
        offsets[0] = 0;
        if (sh[E - 1] > capacity_rows && error_flag) atomicExch(error_flag, 3);   // permuted buffer too small for this routing
    }
}

// ------------------------------------------------------------------------------------------ permute
// One block per token: each of its K copies claims a row inside its expert's padded range and the token's row is copied there.
__global__ void __launch_bounds__(256) moe_permute_kernel(const bf16* __restrict__ x, const int* __restrict__ topk_idx, const int* __restrict__ offsets,
                                                          int* __restrict__ cursors, int* __restrict__ row_map, bf16* __restrict__ xp, int C, int K,
                                                          int expert_base, int num_local, int capacity_rows) {
    __shared__ int rows[16];
    const int tok = blockIdx.x;
    if (threadIdx.x < K) {
        const int e = topk_idx[tok * K + threadIdx.x] - expert_base;
        int r = -1;
        if (e >= 0 && e < num_local) {
            r = offsets[e] + atomicAdd(&cursors[e], 1);
            if (r >= capacity_rows) r = -1;
        }
        rows[threadIdx.x] = r;
        row_map[tok * K + threadIdx.x] = r;
    }
    __syncthreads();
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(tok) * C);
    for (int c = threadIdx.x; c < C / 8; c += blockDim.x) {
        const uint4 v = src[c];
        for (int k = 0; k < K; ++k)
            if (rows[k] >= 0) reinterpret_cast<uint4*>(xp + static_cast<size_t>(rows[k]) * C)[c] = v;
    }
}

// ------------------------------------------------------------------------------------------ un-permute (weighted combine)
// y[token] = sum_k w[token,k] * yp[row_map[token,k]]   (w == nullptr: plain sum, used for permute backward)
__global__ void __launch_bounds__(256) moe_unpermute_kernel(const bf16* __restrict__ yp, const float* __restrict__ w, const int* __restrict__ row_map,
                                                            bf16* __restrict__ y, int C, int K) {
    __shared__ int rows[16];
    __shared__ float ws[16];
    const int tok = blockIdx.x;
    if (threadIdx.x < K) {
        rows[threadIdx.x] = row_map[tok * K + threadIdx.x];
        ws[threadIdx.x] = w ? w[tok * K + threadIdx.x] : 1.f;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C / 8; c += blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < K; ++k) {
            if (rows[k] < 0) continue;
            const uint4 v = reinterpret_cast<const uint4*>(yp + static_cast<size_t>(rows[k]) * C)[c];
            const bf162* p = reinterpret_cast<const bf162*>(&v);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(p[i]);
                acc[2 * i] += ws[k] * f.x;
                acc[2 * i + 1] += ws[k] * f.y;
            }
        }
        uint4 o;
        bf162* po = reinterpret_cast<bf162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        reinterpret_cast<uint4*>(y + static_cast<size_t>(tok) * C)[c] = o;
    }
}

// backward of the weighted combine: d_yp[row] = w * dy[token] ; d_w[token,k] = <yp[row], dy[token]>
__global__ void __launch_bounds__(256) moe_unpermute_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ yp, const float* __restrict__ w,
                                                                const int* __restrict__ row_map, bf16* __restrict__ d_yp, float* __restrict__ d_w,
                                                                int C, int K) {
    __shared__ int rows[16];
    __shared__ float ws[16];
    __shared__ float red[16][8];
    const int tok = blockIdx.x;
    if (threadIdx.x < K) {
        rows[threadIdx.x] = row_map[tok * K + threadIdx.x];
        ws[threadIdx.x] = w[tok * K + threadIdx.x];
    }
    __syncthreads();
    float dots[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) dots[k] = 0.f;
    for (int c = threadIdx.x; c < C / 8; c += blockDim.x) {
        const uint4 gv = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(tok) * C)[c];
        const bf162* gp = reinterpret_cast<const bf162*>(&gv);
        float g[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(gp[i]); g[2 * i] = f.x; g[2 * i + 1] = f.y; }
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            if (k >= K || rows[k] < 0) continue;
            const uint4 v = reinterpret_cast<const uint4*>(yp + static_cast<size_t>(rows[k]) * C)[c];
            const bf162* p = reinterpret_cast<const bf162*>(&v);
            uint4 o;
            bf162* po = reinterpret_cast<bf162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(p[i]);
                dots[k] += f.x * g[2 * i] + f.y * g[2 * i + 1];
                po[i] = __floats2bfloat162_rn(ws[k] * g[2 * i], ws[k] * g[2 * i + 1]);
            }
            reinterpret_cast<uint4*>(d_yp + static_cast<size_t>(rows[k]) * C)[c] = o;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        if (k >= K) break;
        const float s = wsum(dots[k]);
        if (lane == 0) red[k][warp] = s;
    }
    __syncthreads();
    if (threadIdx.x < K) {
        float s = 0.f;
        for (int i = 0; i < (blockDim.x >> 5); ++i) s += red[threadIdx.x][i];
        d_w[tok * K + threadIdx.x] = rows[threadIdx.x] >= 0 ? s : 0.f;
    }
}

// ============================================================================================ launchers
void moe_softmax_topk(const float* logits, float* topk_w, int* topk_idx, float* probs_out, int* counts, float* prob_sum, float* lse_sq_sum,
                      int tokens, int E, int K, int renorm, int num_sms, cudaStream_t s) {
    int grid = (tokens + 7) / 8;
    if (grid > num_sms * 8) grid = num_sms * 8;
    const size_t smem = static_cast<size_t>(E) * 8;
    if (E <= 32) moe_softmax_topk_kernel<1><<<grid, 256, smem, s>>>(logits, topk_w, topk_idx, probs_out, counts, prob_sum, lse_sq_sum, tokens, E, K, renorm);
    else if (E <= 64) moe_softmax_topk_kernel<2><<<grid, 256, smem, s>>>(logits, topk_w, topk_idx, probs_out, counts, prob_sum, lse_sq_sum, tokens, E, K, renorm);
    else if (E <= 128) moe_softmax_topk_kernel<4><<<grid, 256, smem, s>>>(logits, topk_w, topk_idx, probs_out, counts, prob_sum, lse_sq_sum, tokens, E, K, renorm);
    else moe_softmax_topk_kernel<8><<<grid, 256, smem, s>>>(logits, topk_w, topk_idx, probs_out, counts, prob_sum, lse_sq_sum, tokens, E, K, renorm);
}
void moe_offsets(const int* counts, int* offsets, int* cursors, int E, int capacity_rows, int* error_flag, cudaStream_t s) {
    moe_offsets_kernel<<<1, 256, 0, s>>>(counts, offsets, cursors, E, capacity_rows, error_flag);
}
void moe_permute(const void* x, const int* topk_idx, const int* offsets, int* cursors, int* row_map, void* xp, int tokens, int C, int K,
                 int expert_base, int num_local, int capacity_rows, cudaStream_t s) {
    moe_permute_kernel<<<tokens, 256, 0, s>>>((const bf16*)x, topk_idx, offsets, cursors, row_map, (bf16*)xp, C, K, expert_base, num_local, capacity_rows);
}
void moe_unpermute(const void* yp, const float* w, const int* row_map, void* y, int tokens, int C, int K, cudaStream_t s) {
    moe_unpermute_kernel<<<tokens, 256, 0, s>>>((const bf16*)yp, w, row_map, (bf16*)y, C, K);
}
void moe_unpermute_bwd(const void* dy, const void* yp, const float* w, const int* row_map, void* d_yp, float* d_w, int tokens, int C, int K,
                       cudaStream_t s) {
    moe_unpermute_bwd_kernel<<<tokens, 256, 0, s>>>((const bf16*)dy, (const bf16*)yp, w, row_map, (bf16*)d_yp, d_w, C, K);
}

void moe_router_bwd(const float* logits, const int* topk_idx, const float* d_topk_w, const int* counts, const float* d_aux, void* d_logits, int tokens,
                    int E, int K, int renorm, float aux_coef, float z_coef, int num_sms, cudaStream_t s) {
    const int blocks = min((tokens + 7) / 8, num_sms * 8);
#define SG_RB(V) moe_router_bwd_kernel<V><<<blocks, 256, 0, s>>>(logits, topk_idx, d_topk_w, counts, d_aux, (bf16*)d_logits, tokens, E, K, renorm, aux_coef, z_coef)
    if (E <= 32) SG_RB(1); else if (E <= 64) SG_RB(2); else if (E <= 128) SG_RB(4); else SG_RB(8);
#undef SG_RB
}

}  // namespace sg

// Causal flash attention with grouped-query heads for sm_100a (head_dim 128, bf16), on tcgen05 tensor cores.
//
// Input is the packed projection output [B, T, (Hq + 2*Hkv) * 128] (queries, then keys, then values; rotary and QK-norm
// already applied).  The kernels read Q/K/V tiles straight out of that tensor with TMA: no split or transpose copies.
//
// Forward (one CTA per 128-query tile of one head):
//   warp 0      TMA producer: Q once, then K_j / V_j tiles through a 2-stage ring
//   warp 1      MMA issuer:   S_j = Q K_j^T  into one of two TMEM score buffers, then O += P_j V_j (V read MN-major)
//   warps 2-5   softmax:      thread r owns query row r: reads S_j from TMEM, online softmax in base 2, writes P_j (bf16) to
//                             shared memory in the 128-byte-swizzled K-major layout the second MMA reads; the running
//                             output in TMEM is rescaled only when a row maximum grew by more than 2^8 (exact, but rare)
//   S_{j+1} is issued before P_j V_j, so the score MMA overlaps the softmax of the previous tile.
//
// Backward is two kernels that recompute the scores (nothing but O and the log-sum-exp is kept from forward):
//   dK/dV kernel: one CTA per 128-key tile of one KV head, loops over the query tiles of the G query heads that share it:
//                 S^T = K Q^T, dP^T = V dO^T, P^T = exp2(S^T - lse), dS^T = P^T o (dP^T - delta); dV += P^T dO, dK += dS^T Q
//                 (the GQA reduction happens in the TMEM accumulators, no atomics)
//   dQ kernel:    one CTA per 128-query tile of one head, loops over key tiles: dQ += dS K
//
// Every mbarrier wait is bounded (error word + clean exit).  Replaces the cuDNN SDPA graph and the FlashAttention-2
// kernels of the reference (csrc/src/runtime/attention/backend_cudnn.cpp, backend_flash_varlen.cpp).
#include <cuda_bf16.h>
#include <math_constants.h>

#include "attention_sm100.h"
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace sg {
namespace fa {

constexpr int BQ = 128, BKV = 128, D = 128;
constexpr int TILE_BYTES = 128 * D * 2;        // 32 KB: 128 rows x 128 bf16, stored as two 16 KB halves of 64 columns
constexpr int HALF = 16384;
constexpr int THREADS = 192;
constexpr float RESCALE_THRESHOLD = 8.f;       // log2 units

__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t unit16) { return row * 128u + ((unit16 ^ (row & 7u)) << 4); }

// S (or any 128x128 result) = A[128, 128] . B[128, 128]^T, both K-major tiles (two 64-column halves): 8 MMAs of K = 16
__device__ __forceinline__ void mma_kk(uint32_t d_tmem, uint32_t a_base, uint32_t b_base, uint32_t idesc, bool accumulate_first) {
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint64_t da = make_smem_desc(a_base + c * HALF + ks * 32, 16, 1024);
            const uint64_t db = make_smem_desc(b_base + c * HALF + ks * 32, 16, 1024);
            mma_f16(d_tmem, da, db, idesc, (accumulate_first || c > 0 || ks > 0) ? 1u : 0u);
        }
}
// D[128, 128] (+)= A[128 x 128 contraction] (K-major) . B where B is stored [contraction rows][128 columns] (MN-major)
__device__ __forceinline__ void mma_k_mn(uint32_t d_tmem, uint32_t a_base, uint32_t b_base, uint32_t idesc, bool accumulate_first) {
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint64_t da = make_smem_desc(a_base + c * HALF + ks * 32, 16, 1024);
            const uint64_t db = make_smem_desc(b_base + (c * 4 + ks) * 2048, HALF, 1024);
            mma_f16(d_tmem, da, db, idesc, (accumulate_first || c > 0 || ks > 0) ? 1u : 0u);
        }
}

__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* tm, int col, int row, uint32_t bar) {
    tma_load_2d(dst, tm, col, row, bar);
    tma_load_2d(dst + HALF, tm, col + 64, row, bar);
}

// write 32 consecutive values of row `row` (columns [c0, c0+32)) as bf16 into a K-major swizzled 128x128 tile
__device__ __forceinline__ void store_row32(uint8_t* tile, int row, int c0, const float (&v)[32]) {
    uint8_t* half = tile + (c0 >> 6) * HALF;
    const int u0 = (c0 & 63) >> 3;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        uint4 o;
        __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(v[u * 8 + 2 * i], v[u * 8 + 2 * i + 1]);
        *reinterpret_cast<uint4*>(half + swz(row, u0 + u)) = o;
    }
}

struct FwdParams {
    __nv_bfloat16* out;   // [B, T, Hq*128]
    float* lse;           // [B, T, Hq]   natural-log sum-exp of the scaled scores
    int T, Hq, Hkv;
    float scale_log2;     // softmax_scale * log2(e)
    int* error_flag;
};

__global__ void __launch_bounds__(THREADS, 1) fa_fwd_kernel(const __grid_constant__ CUtensorMap tm, const FwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_q = smem_u32(smem), s_kv = s_q + TILE_BYTES, s_p = s_kv + 4 * TILE_BYTES;
    uint8_t* p_tile = smem + 5 * TILE_BYTES;
    const uint32_t bars = s_p + TILE_BYTES;
    // barriers: 0 q_full | 1,2 kv_full | 3,4 kv_empty | 5,6 s_full | 7,8 s_empty | 9 p_full | 10 p_empty | 11 o_full
    auto bar = [&](int i) { return bars + 8u * i; };
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_blk = gridDim.x - 1 - blockIdx.x;   // long (late) query tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.Hq / p.Hkv);
    const int n_kv = q_blk + 1;
    const int row0 = b * p.T;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(bar(0), 1);
        for (int i = 1; i <= 8; ++i) mbar_init(bar(i), (i == 7 || i == 8) ? 128 : 1);
        mbar_init(bar(9), 128);
        mbar_init(bar(10), 1);
        mbar_init(bar(11), 1);
        fence_barrier_init();
        tma_prefetch_desc(&tm);
    }
    if (warp == 2) { tmem_alloc(smem_u32(&tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t t_s[2] = {tmem, tmem + 128}, t_o = tmem + 256;

    if (warp == 0) {
        if (elect_one()) {
            mbar_expect_tx(bar(0), TILE_BYTES);
            load_tile(s_q, &tm, h * D, row0 + q_blk * BQ, bar(0));
            for (int j = 0; j < n_kv; ++j) {
                const int st = j & 1;
                if (!mbar_wait(bar(3 + st), ((j >> 1) & 1) ^ 1u, &abort_flag)) break;
                mbar_expect_tx(bar(1 + st), 2 * TILE_BYTES);
                load_tile(s_kv + st * 2 * TILE_BYTES, &tm, (p.Hq + hk) * D, row0 + j * BKV, bar(1 + st));
                load_tile(s_kv + st * 2 * TILE_BYTES + TILE_BYTES, &tm, (p.Hq + p.Hkv + hk) * D, row0 + j * BKV, bar(1 + st));
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc_s = make_idesc(1, 1, 0, 0, 128, 128);
            const uint32_t idesc_pv = make_idesc(1, 1, 0, 1, 128, 128);
            bool ok = mbar_wait(bar(0), 0, &abort_flag);
            for (int j = 0; j < n_kv && ok; ++j) {
                const int st = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                if (!mbar_wait(bar(1 + st), ph, &abort_flag)) { ok = false; break; }
                if (!mbar_wait(bar(7 + st), ph ^ 1u, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                mma_kk(t_s[st], s_q, s_kv + st * 2 * TILE_BYTES, idesc_s, false);
                tc_commit(bar(5 + st));
                if (j >= 1) {
                    if (!mbar_wait(bar(9), (j - 1) & 1, &abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const int pst = (j - 1) & 1;
                    mma_k_mn(t_o, s_p, s_kv + pst * 2 * TILE_BYTES + TILE_BYTES, idesc_pv, j - 1 > 0);
                    tc_commit(bar(3 + pst));
                    tc_commit(bar(10));
                }
            }
            if (ok && mbar_wait(bar(9), (n_kv - 1) & 1, &abort_flag)) {
                tc_fence_after();
                const int pst = (n_kv - 1) & 1;
                mma_k_mn(t_o, s_p, s_kv + pst * 2 * TILE_BYTES + TILE_BYTES, idesc_pv, n_kv - 1 > 0);
                tc_commit(bar(3 + pst));
                tc_commit(bar(10));
                tc_commit(bar(11));
            }
        }
    } else {
        const int quad = warp & 3;
        const int r = quad * 32 + lane;                       // query row inside the tile
        const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
        float m_used = -CUDART_INF_F, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kv && ok; ++j) {
            const int st = j & 1;
            if (!mbar_wait(bar(5 + st), (j >> 1) & 1, &abort_flag)) { ok = false; break; }
            tc_fence_after();
            float s[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t raw[32];
                tmem_ld_32x32(t_s[st] + lane_sel + c * 32, raw);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(raw[i]) * p.scale_log2;
            }
            tc_fence_before();
            mbar_arrive(bar(7 + st));                         // score buffer may be overwritten by S_{j+2}
            if (j == q_blk) {                                  // diagonal tile: keys after the query are masked
#pragma unroll
                for (int i = 0; i < 128; ++i)
                    if (i > r) s[i] = -CUDART_INF_F;
            }
            float m_blk = s[0];
#pragma unroll
            for (int i = 1; i < 128; ++i) m_blk = fmaxf(m_blk, s[i]);
            const bool grow = m_blk > m_used + RESCALE_THRESHOLD;   // first tile: m_used = -inf -> true
            if (j > 0) {
                if (!mbar_wait(bar(10), (j - 1) & 1, &abort_flag)) { ok = false; break; }   // P buffer free, O stable
                tc_fence_after();
                if (__any_sync(0xffffffffu, grow)) {
                    const float f = grow ? exp2f(m_used - m_blk) : 1.f;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t raw[32];
                        tmem_ld_32x32(t_o + lane_sel + c * 32, raw);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * f);
                        tmem_st_32x32(t_o + lane_sel + c * 32, raw);
                    }
                    tmem_st_wait();
                    l *= f;
                }
            }
            if (grow) m_used = m_blk;
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float pv[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) { pv[i] = exp2f(s[c * 32 + i] - m_used); sum += pv[i]; }
                store_row32(p_tile, r, c * 32, pv);
            }
            l += sum;
            fence_proxy_async();                               // generic-proxy writes of P -> visible to the tensor core
            tc_fence_before();
            mbar_arrive(bar(9));
        }
        if (ok && mbar_wait(bar(11), 0, &abort_flag)) {
            tc_fence_after();
            const float inv = 1.f / l;
            __nv_bfloat16* orow = p.out + (static_cast<size_t>(row0 + q_blk * BQ + r) * p.Hq + h) * D;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t raw[32];
                tmem_ld_32x32(t_o + lane_sel + c * 32, raw);
                tmem_ld_wait();
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    uint4 o;
                    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        po[i] = __floats2bfloat162_rn(__uint_as_float(raw[u * 8 + 2 * i]) * inv, __uint_as_float(raw[u * 8 + 2 * i + 1]) * inv);
                    *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = o;
                }
            }
            p.lse[static_cast<size_t>(row0 + q_blk * BQ + r) * p.Hq + h] = (m_used + log2f(l)) * 0.6931471805599453f;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag && p.error_flag) atomicExch(p.error_flag, 4);
    if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

constexpr int FWD_SMEM = 6 * TILE_BYTES + 1024 + 256;

// ------------------------------------------------------------------------------------------------ backward
// delta[b, t, h] = sum_d dO * O   (one warp per (token, head))
__global__ void __launch_bounds__(256) fa_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                                                       size_t items) {
    const int lane = threadIdx.x & 31;
    for (size_t it = blockIdx.x * static_cast<size_t>(blockDim.x >> 5) + (threadIdx.x >> 5); it < items; it += static_cast<size_t>(gridDim.x) * (blockDim.x >> 5)) {
        const uint2 a = *reinterpret_cast<const uint2*>(o + it * D + lane * 4), g = *reinterpret_cast<const uint2*>(d_o + it * D + lane * 4);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* pg = reinterpret_cast<const __nv_bfloat162*>(&g);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pg[i]);
            s += x.x * y.x + x.y * y.y;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lane == 0) delta[it] = s;
    }
}

struct BwdParams {
    __nv_bfloat16* d_qkv;   // [B, T, (Hq+2Hkv)*128]
    const float* lse;       // [B, T, Hq] natural log
    const float* delta;     // [B, T, Hq]
    int T, Hq, Hkv;
    float scale, scale_log2;
    int* error_flag;
};

// write a finished 128x128 fp32 TMEM accumulator as bf16 rows of the packed gradient tensor
__device__ __forceinline__ void store_acc_rows(uint32_t t_acc, uint32_t lane_sel, __nv_bfloat16* dst_row, float mul) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(t_acc + lane_sel + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            uint4 o;
            __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                po[i] = __floats2bfloat162_rn(__uint_as_float(raw[u * 8 + 2 * i]) * mul, __uint_as_float(raw[u * 8 + 2 * i + 1]) * mul);
            *reinterpret_cast<uint4*>(dst_row + c * 32 + u * 8) = o;
        }
    }
}

// dK / dV: one CTA per (key tile, KV head, batch)
__global__ void __launch_bounds__(THREADS, 1) fa_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                                                                const BwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_k = smem_u32(smem), s_v = s_k + TILE_BYTES, s_q = s_v + TILE_BYTES, s_do = s_q + TILE_BYTES, s_pt = s_do + TILE_BYTES,
                   s_dst = s_pt + TILE_BYTES;
    uint8_t* pt_tile = smem + 4 * TILE_BYTES;
    uint8_t* dst_tile = smem + 5 * TILE_BYTES;
    const uint32_t bars = s_dst + TILE_BYTES;
    float* vec = reinterpret_cast<float*>(smem + 6 * TILE_BYTES + 128);   // [2][2][128]: (buffer, lse2|delta, query)
    auto bar = [&](int i) { return bars + 8u * i; };
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int G = p.Hq / p.Hkv, nq = p.T / BQ;
    const int per_head = nq - kb;            // query tiles at or after this key tile
    const int n_items = G * per_head;
    const int row0 = b * p.T;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(bar(0), 1); mbar_init(bar(1), 1); mbar_init(bar(2), 1); mbar_init(bar(3), 1);
        mbar_init(bar(4), 128); mbar_init(bar(5), 128); mbar_init(bar(6), 1); mbar_init(bar(7), 128);
        fence_barrier_init();
        tma_prefetch_desc(&tm_qkv);
        tma_prefetch_desc(&tm_do);
    }
    if (warp == 2) { tmem_alloc(smem_u32(&tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t t_st = tmem, t_dpt = tmem + 128, t_dv = tmem + 256, t_dk = tmem + 384;

    if (warp == 0) {
        if (elect_one()) {
            mbar_expect_tx(bar(0), 2 * TILE_BYTES);
            load_tile(s_k, &tm_qkv, (p.Hq + hk) * D, row0 + kb * BKV, bar(0));
            load_tile(s_v, &tm_qkv, (p.Hq + p.Hkv + hk) * D, row0 + kb * BKV, bar(0));
            for (int i = 0; i < n_items; ++i) {
                const int h = hk * G + i / per_head, qb = kb + i % per_head;
                if (!mbar_wait(bar(2), (i & 1) ^ 1u, &abort_flag)) break;
                mbar_expect_tx(bar(1), 2 * TILE_BYTES);
                load_tile(s_q, &tm_qkv, h * D, row0 + qb * BQ, bar(1));
                load_tile(s_do, &tm_do, h * D, row0 + qb * BQ, bar(1));
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc_kk = make_idesc(1, 1, 0, 0, 128, 128), idesc_kmn = make_idesc(1, 1, 0, 1, 128, 128);
            bool ok = mbar_wait(bar(0), 0, &abort_flag);
            for (int i = 0; i < n_items && ok; ++i) {
                if (!mbar_wait(bar(1), i & 1, &abort_flag)) { ok = false; break; }
                if (!mbar_wait(bar(4), (i & 1) ^ 1u, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                mma_kk(t_st, s_k, s_q, idesc_kk, false);      // S^T  = K Q^T
                mma_kk(t_dpt, s_v, s_do, idesc_kk, false);    // dP^T = V dO^T
                tc_commit(bar(3));
                if (!mbar_wait(bar(5), i & 1, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                mma_k_mn(t_dv, s_pt, s_do, idesc_kmn, i > 0);  // dV += P^T dO
                mma_k_mn(t_dk, s_dst, s_q, idesc_kmn, i > 0);  // dK += dS^T Q
                tc_commit(bar(2));
            }
            if (ok) tc_commit(bar(6));
        }
    } else {
        const int quad = warp & 3;
        const int r = quad * 32 + lane;     // key row inside the tile
        const int t = (warp - 2) * 32 + lane;
        const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
        bool ok = true;
        for (int i = 0; i < n_items && ok; ++i) {
            const int h = hk * G + i / per_head, qb = kb + i % per_head;
            float* lse2 = vec + (i & 1) * 256;
            float* dl = lse2 + 128;
            {
                const size_t idx = static_cast<size_t>(row0 + qb * BQ + t) * p.Hq + h;
                lse2[t] = p.lse[idx] * 1.4426950408889634f;
                dl[t] = p.delta[idx];
            }
            mbar_arrive(bar(7));                                                         // all 128 entries of this item's vectors are written
            if (!mbar_wait(bar(7), i & 1, &abort_flag)) { ok = false; break; }
            if (!mbar_wait(bar(3), i & 1, &abort_flag)) { ok = false; break; }
            if (!mbar_wait(bar(2), (i & 1) ^ 1u, &abort_flag)) { ok = false; break; }   // previous item's MMAs no longer read P^T / dS^T
            tc_fence_after();
            const bool diag = qb == kb;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t rs[32], rd[32];
                tmem_ld_32x32(t_st + lane_sel + c * 32, rs);
                tmem_ld_32x32(t_dpt + lane_sel + c * 32, rd);
                tmem_ld_wait();
                float pv[32], ds[32];
#pragma unroll
                for (int k = 0; k < 32; ++k) {
                    const int qc = c * 32 + k;   // query column
                    float pr = ex2_approx(fmaf(__uint_as_float(rs[k]), p.scale_log2, -lse2[qc]));
                    if (diag && r > qc) pr = 0.f;
                    pv[k] = pr;
                    ds[k] = pr * (__uint_as_float(rd[k]) - dl[qc]) * p.scale;
                }
                store_row32(pt_tile, r, c * 32, pv);
                store_row32(dst_tile, r, c * 32, ds);
            }
            tc_fence_before();
            mbar_arrive(bar(4));
            fence_proxy_async();
            mbar_arrive(bar(5));
        }
        if (ok && mbar_wait(bar(6), 0, &abort_flag)) {
            tc_fence_after();
            const size_t width = static_cast<size_t>(p.Hq + 2 * p.Hkv) * D;
            __nv_bfloat16* base = p.d_qkv + static_cast<size_t>(row0 + kb * BKV + r) * width;
            store_acc_rows(t_dk, lane_sel, base + (p.Hq + hk) * D, 1.f);
            store_acc_rows(t_dv, lane_sel, base + (p.Hq + p.Hkv + hk) * D, 1.f);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag && p.error_flag) atomicExch(p.error_flag, 5);
    if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// dQ: one CTA per (query tile, head, batch)
__global__ void __launch_bounds__(THREADS, 1) fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                                                               const BwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_q = smem_u32(smem), s_do = s_q + TILE_BYTES, s_k = s_do + TILE_BYTES, s_v = s_k + TILE_BYTES, s_ds = s_v + TILE_BYTES;
    uint8_t* ds_tile = smem + 4 * TILE_BYTES;
    const uint32_t bars = s_ds + TILE_BYTES;
    auto bar = [&](int i) { return bars + 8u * i; };
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_blk = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.Hq / p.Hkv);
    const int n_kv = q_blk + 1;
    const int row0 = b * p.T;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(bar(0), 1); mbar_init(bar(1), 1); mbar_init(bar(2), 1); mbar_init(bar(3), 1);
        mbar_init(bar(4), 128); mbar_init(bar(5), 128); mbar_init(bar(6), 1);
        fence_barrier_init();
        tma_prefetch_desc(&tm_qkv);
        tma_prefetch_desc(&tm_do);
    }
    if (warp == 2) { tmem_alloc(smem_u32(&tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t t_s = tmem, t_dp = tmem + 128, t_dq = tmem + 256;

    if (warp == 0) {
        if (elect_one()) {
            mbar_expect_tx(bar(0), 2 * TILE_BYTES);
            load_tile(s_q, &tm_qkv, h * D, row0 + q_blk * BQ, bar(0));
            load_tile(s_do, &tm_do, h * D, row0 + q_blk * BQ, bar(0));
            for (int j = 0; j < n_kv; ++j) {
                if (!mbar_wait(bar(2), (j & 1) ^ 1u, &abort_flag)) break;
                mbar_expect_tx(bar(1), 2 * TILE_BYTES);
                load_tile(s_k, &tm_qkv, (p.Hq + hk) * D, row0 + j * BKV, bar(1));
                load_tile(s_v, &tm_qkv, (p.Hq + p.Hkv + hk) * D, row0 + j * BKV, bar(1));
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc_kk = make_idesc(1, 1, 0, 0, 128, 128), idesc_kmn = make_idesc(1, 1, 0, 1, 128, 128);
            bool ok = mbar_wait(bar(0), 0, &abort_flag);
            for (int j = 0; j < n_kv && ok; ++j) {
                if (!mbar_wait(bar(1), j & 1, &abort_flag)) { ok = false; break; }
                if (!mbar_wait(bar(4), (j & 1) ^ 1u, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                mma_kk(t_s, s_q, s_k, idesc_kk, false);       // S  = Q K^T
                mma_kk(t_dp, s_do, s_v, idesc_kk, false);     // dP = dO V^T
                tc_commit(bar(3));
                if (!mbar_wait(bar(5), j & 1, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                mma_k_mn(t_dq, s_ds, s_k, idesc_kmn, j > 0);   // dQ += dS K
                tc_commit(bar(2));
            }
            if (ok) tc_commit(bar(6));
        }
    } else {
        const int quad = warp & 3;
        const int r = quad * 32 + lane;     // query row
        const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
        const size_t idx = static_cast<size_t>(row0 + q_blk * BQ + r) * p.Hq + h;
        const float lse2 = p.lse[idx] * 1.4426950408889634f, dl = p.delta[idx];
        bool ok = true;
        for (int j = 0; j < n_kv && ok; ++j) {
            if (!mbar_wait(bar(3), j & 1, &abort_flag)) { ok = false; break; }
            if (!mbar_wait(bar(2), (j & 1) ^ 1u, &abort_flag)) { ok = false; break; }
            tc_fence_after();
            const bool diag = j == q_blk;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t rs[32], rd[32];
                tmem_ld_32x32(t_s + lane_sel + c * 32, rs);
                tmem_ld_32x32(t_dp + lane_sel + c * 32, rd);
                tmem_ld_wait();
                float ds[32];
#pragma unroll
                for (int k = 0; k < 32; ++k) {
                    const int kc = c * 32 + k;   // key column
                    float pr = ex2_approx(fmaf(__uint_as_float(rs[k]), p.scale_log2, -lse2));
                    if (diag && kc > r) pr = 0.f;
                    ds[k] = pr * (__uint_as_float(rd[k]) - dl) * p.scale;
                }
                store_row32(ds_tile, r, c * 32, ds);
            }
            tc_fence_before();
            mbar_arrive(bar(4));
            fence_proxy_async();
            mbar_arrive(bar(5));
        }
        if (ok && mbar_wait(bar(6), 0, &abort_flag)) {
            tc_fence_after();
            const size_t width = static_cast<size_t>(p.Hq + 2 * p.Hkv) * D;
            store_acc_rows(t_dq, lane_sel, p.d_qkv + static_cast<size_t>(row0 + q_blk * BQ + r) * width + h * D, 1.f);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag && p.error_flag) atomicExch(p.error_flag, 6);
    if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

constexpr int DKV_SMEM = 6 * TILE_BYTES + 128 + 2048 + 1024;
constexpr int DQ_SMEM = 5 * TILE_BYTES + 256 + 1024;

}  // namespace fa

const char* flash_attn_fwd_sm100(const void* qkv, void* out, float* lse, int B, int T, int Hq, int Hkv, float softmax_scale, int* error_flag,
                                 cudaStream_t stream) {
    using namespace fa;
    if (T % 128 != 0) return "flash_attn_fwd: T must be a multiple of 128";
    if (Hq % Hkv != 0) return "flash_attn_fwd: Hq must be a multiple of Hkv";
    CUtensorMap tm;
    const uint64_t width = static_cast<uint64_t>(Hq + 2 * Hkv) * D;
    const char* e = make_tensor_map_2d(&tm, qkv, 2, width, static_cast<uint64_t>(B) * T, width * 2, 64, 128);
    if (e) return e;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(fa_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM) != cudaSuccess)
            return "cudaFuncSetAttribute failed (flash_attn_fwd)";
        attr_set = true;
    }
    FwdParams p{static_cast<__nv_bfloat16*>(out), lse, T, Hq, Hkv, softmax_scale * 1.4426950408889634f, error_flag};
    fa_fwd_kernel<<<dim3(T / 128, Hq, B), THREADS, FWD_SMEM, stream>>>(tm, p);
    return cudaGetLastError() == cudaSuccess ? nullptr : "flash_attn_fwd launch failed";
}

const char* flash_attn_bwd_sm100(const void* qkv, const void* out, const void* d_out, const float* lse, float* delta, void* d_qkv, int B, int T, int Hq,
                                 int Hkv, float softmax_scale, int* error_flag, int num_sms, cudaStream_t stream, int variant) {
    using namespace fa;
    if (T % 128 != 0) return "flash_attn_bwd: T must be a multiple of 128";
    CUtensorMap tm_qkv, tm_do;
    const uint64_t width = static_cast<uint64_t>(Hq + 2 * Hkv) * D, owidth = static_cast<uint64_t>(Hq) * D;
    const char* e = make_tensor_map_2d(&tm_qkv, qkv, 2, width, static_cast<uint64_t>(B) * T, width * 2, 64, 128);
    if (e) return e;
    e = make_tensor_map_2d(&tm_do, d_out, 2, owidth, static_cast<uint64_t>(B) * T, owidth * 2, 64, 128);
    if (e) return e;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(fa_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DKV_SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(fa_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM) != cudaSuccess)
            return "cudaFuncSetAttribute failed (flash_attn_bwd)";
        attr_set = true;
    }
    const size_t items = static_cast<size_t>(B) * T * Hq;
    int grid = static_cast<int>((items + 7) / 8);
    if (grid > num_sms * 8) grid = num_sms * 8;
    fa_delta_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(d_out), delta, items);
    if (variant != 128) return flash_attn_bwd64_sm100(qkv, d_out, lse, delta, d_qkv, B, T, Hq, Hkv, softmax_scale, error_flag, stream);
    BwdParams p{static_cast<__nv_bfloat16*>(d_qkv), lse, delta, T, Hq, Hkv, softmax_scale, softmax_scale * 1.4426950408889634f, error_flag};
    fa_bwd_dkv_kernel<<<dim3(T / 128, Hkv, B), THREADS, DKV_SMEM, stream>>>(tm_qkv, tm_do, p);
    fa_bwd_dq_kernel<<<dim3(T / 128, Hq, B), THREADS, DQ_SMEM, stream>>>(tm_qkv, tm_do, p);
    return cudaGetLastError() == cudaSuccess ? nullptr : "flash_attn_bwd launch failed";
}

}  // namespace sg

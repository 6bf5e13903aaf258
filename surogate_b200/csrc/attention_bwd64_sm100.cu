// Flash-attention backward (causal, GQA, head_dim 128; nothing but O and the log-sum-exp is kept from forward, scores are recomputed):
//
// One kernel template serves both passes.  A CTA keeps a RESIDENT pair of 128-row tiles and streams 64-row tile pairs through
// a 3-stage TMA ring; two score accumulators (X = R1 . S1^T, Y = R2 . S2^T) are double-buffered in TMEM so the MMAs of item
// i+1 run while the softmax warps still work on item i; the gradient accumulators stay in TMEM for the whole CTA.
//   dK/dV pass: resident (K, V) of one 128-key tile of one KV head, streamed (Q, dO) tiles of the G query heads that share it:
//               X = S^T, Y = dP^T, P^T = exp2(S^T - lse), dS^T = P^T o (dP^T - delta); dV += P^T dO, dK += dS^T Q.
//   dQ pass   : resident (Q, dO) of one 128-query tile, streamed (K, V) tiles: X = S, Y = dP, dS = P o (dP - delta); dQ += dS K.
// The GQA reduction of dK / dV happens in the TMEM accumulators (no atomics).  Every mbarrier wait is bounded.
// Optional per-row lower bound `lo[b, t]` (HAS_LO; packed documents and sliding windows, see attention_fwd64_sm100.cu): the dQ pass
// starts at key tile lo[first query] / 64; the dK/dV pass stops at `kv_qend[b, key tile]`, the first 64-row query tile in which no
// query can see the key tile any more (lo is non-decreasing, so that is one number per key tile).
#include <cuda_bf16.h>
#include <math_constants.h>

#include "attention_sm100.h"
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace sg {
namespace fb64 {

constexpr int D = 128;
constexpr int T128 = 128 * D * 2;     // 32 KB tile of 128 rows: two halves of 16 KB
constexpr int H128 = 16384;
constexpr int T64 = 64 * D * 2;       // 16 KB tile of 64 rows: two halves of 8 KB
constexpr int H64 = 8192;
constexpr int ROWS128x64 = 128 * 128; // 16 KB: 128 rows x 64 bf16 (one 128-byte swizzled row each)
constexpr int THREADS = 320;      // TMA warp, MMA warp, 8 softmax warps (two per TMEM lane quadrant, 32 of the 64 columns each)
constexpr float LOG2E = 1.4426950408889634f;

struct Params {
    __nv_bfloat16* d_qkv;
    const float* lse;
    const float* delta;
    int T, Hq, Hkv;
    float scale, scale_log2;
    int* error_flag;
    long long* prof;   // optional [16]: per-phase cycle counters of one softmax thread of each pass (development aid)
    const int* lo;       // optional [B, T]: first key each query may attend
    const int* kv_qend;  // with lo: [B, T / 128] exclusive end, in 64-row query tiles, of the queries that attend each 128-key tile
};

#define FB_PROF(k)                                   \
    do {                                             \
        if (do_prof) {                               \
            const long long now_ = clock64();        \
            acc_[k] += now_ - t_;                    \
            t_ = now_;                               \
        }                                            \
    } while (0)

// row `r` of a [128 x 64] bf16 tile (128-byte rows, 16-byte units XOR-swizzled with the row index)
__device__ __forceinline__ void store_row64(uint8_t* tile, int r, const float (&v)[64]) {
    uint8_t* row = tile + r * 128;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        uint4 o;
        __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(v[u * 8 + 2 * i], v[u * 8 + 2 * i + 1]);
        *reinterpret_cast<uint4*>(row + ((u ^ (r & 7)) << 4)) = o;
    }
}
// 32 columns [32*half, 32*half+32) of row `r` of a [128 x 64] swizzled tile
__device__ __forceinline__ void store_row32h(uint8_t* tile, int r, int half, const float (&v)[32]) {
    uint8_t* row = tile + r * 128;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        uint4 o;
        __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(v[u * 8 + 2 * i], v[u * 8 + 2 * i + 1]);
        *reinterpret_cast<uint4*>(row + (((half * 4 + u) ^ (r & 7)) << 4)) = o;
    }
}
__device__ __forceinline__ void ld32f(uint32_t taddr, float (&v)[32]) {
    uint32_t a[32];
    tmem_ld_32x32(taddr, a);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(a[i]);
}
__device__ __forceinline__ void ld64(uint32_t taddr, float (&v)[64]) {
    uint32_t a[32], b[32];
    tmem_ld_32x32(taddr, a);
    tmem_ld_32x32(taddr + 32, b);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) { v[i] = __uint_as_float(a[i]); v[32 + i] = __uint_as_float(b[i]); }
}
// columns [64*half, 64*half+64) of a finished 128x128 fp32 accumulator -> bf16 row in global memory
__device__ __forceinline__ void store_acc128(uint32_t t_acc, uint32_t lane_sel, __nv_bfloat16* dst_row, int half) {
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        uint32_t raw[32];
        tmem_ld_32x32(t_acc + lane_sel + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            uint4 o;
            __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(__uint_as_float(raw[u * 8 + 2 * i]), __uint_as_float(raw[u * 8 + 2 * i + 1]));
            *reinterpret_cast<uint4*>(dst_row + c * 32 + u * 8) = o;
        }
    }
}
// D[128, 64] = A[128 rows, d] . B[64 rows, d]^T  (contraction d = 128: 2 halves x 4 steps)
__device__ __forceinline__ void mma_128x64_kk(uint32_t d_tmem, uint32_t a128, uint32_t b64, uint32_t idesc) {
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
            mma_f16(d_tmem, make_smem_desc(a128 + c * H128 + ks * 32, 16, 1024), make_smem_desc(b64 + c * H64 + ks * 32, 16, 1024), idesc,
                    (c > 0 || ks > 0) ? 1u : 0u);
}
// D[128, 128] (+)= A[128 rows x 64 contraction] (one swizzled 128-byte row each) . B stored [64 contraction rows][128 cols] (two 8 KB halves)
__device__ __forceinline__ void mma_acc_k64(uint32_t d_tmem, uint32_t a_rows, uint32_t b64, uint32_t idesc, bool acc) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
        mma_f16(d_tmem, make_smem_desc(a_rows + ks * 32, 16, 1024), make_smem_desc(b64 + ks * 2048, H64, 1024), idesc, (acc || ks > 0) ? 1u : 0u);
}

// ------------------------------------------------------------------------------------------------ the kernel
// R1 | R2 | ring (S1, S2) x 3 | P(^T) | dS(^T) | barriers | per-item vectors
constexpr int RING = 3;
constexpr int OFF_R2 = T128, OFF_RING = 2 * T128, STAGE = 2 * T64, OFF_PT = OFF_RING + RING * STAGE, OFF_DST = OFF_PT + ROWS128x64,
              OFF_BAR = OFF_DST + ROWS128x64, OFF_VEC = OFF_BAR + 256;
constexpr int OFF_VLO = OFF_VEC + 2 * 2 * 64 * 4;   // per-item lower bounds of the 64 streamed queries (dK/dV pass), double-buffered
constexpr int SMEM = OFF_VLO + 2 * 64 * 4;
// barriers: 0 res_full | 1-3 ring_full | 4-6 ring_empty | 7,8 xy_full | 9,10 xy_free | 11 pds_full | 12 pds_empty | 13 done | 14 vec_full
constexpr int B_RES = 0, B_RFULL = 1, B_REMPTY = 4, B_XY = 7, B_XYFREE = 9, B_PDS = 11, B_PDSE = 12, B_DONE = 13, B_VEC = 14;

template <bool IS_DQ, bool HAS_LO>
__global__ void __launch_bounds__(THREADS, 1) fa_bwd64_kernel(const __grid_constant__ CUtensorMap tm_qkv128, const __grid_constant__ CUtensorMap tm_qkv64,
                                                              const __grid_constant__ CUtensorMap tm_do128, const __grid_constant__ CUtensorMap tm_do64,
                                                              const Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t s0 = smem_u32(smem);
    const uint32_t s_r1 = s0, s_r2 = s0 + OFF_R2, s_ring = s0 + OFF_RING, s_pt = s0 + OFF_PT, s_dst = s0 + OFF_DST, bars = s0 + OFF_BAR;
    uint8_t* pt_tile = smem + OFF_PT;
    uint8_t* dst_tile = smem + OFF_DST;
    float* vec = reinterpret_cast<float*>(smem + OFF_VEC);
    int* vec_lo = reinterpret_cast<int*>(smem + OFF_VLO);
    auto bar = [&](int i) { return bars + 8u * i; };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_BAR + 136);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, row0 = b * p.T;
    const int G = p.Hq / p.Hkv;
    // dK/dV: tile = key tile kb (light-to-heavy order is reversed: early key tiles see the most query tiles), head = KV head
    // dQ   : tile = query tile (late tiles first), head = query head
    const int tile = IS_DQ ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
    const int head = blockIdx.y;
    const int hk = IS_DQ ? head / G : head;
    // streamed 64-row tiles [first_ct, first_ct + per_head): keys from the lower bound of the tile's first query up to the diagonal
    // (dQ), queries from the diagonal to the last one that can still see this key tile (dK/dV)
    const int first_ct = IS_DQ ? (HAS_LO ? __ldg(p.lo + row0 + tile * 128) / 64 : 0) : 2 * tile;
    const int last_ct = IS_DQ ? 2 * (tile + 1) : (HAS_LO ? __ldg(p.kv_qend + b * (p.T / 128) + tile) : p.T / 64);
    const int per_head = last_ct - first_ct;
    const int n_items = IS_DQ ? per_head : G * per_head;
    const int kcol = (p.Hq + hk) * D, vcol = (p.Hq + p.Hkv + hk) * D;

    if (threadIdx.x == 0) {
        *abort_flag = (s0 & 1023u) ? 1 : 0;
        for (int i = 0; i <= 8; ++i) mbar_init(bar(i), 1);
        mbar_init(bar(9), 256); mbar_init(bar(10), 256); mbar_init(bar(B_PDS), 256);
        mbar_init(bar(B_PDSE), 1); mbar_init(bar(B_DONE), 1); mbar_init(bar(B_VEC), 256);
        fence_barrier_init();
    }
    if (warp == 2) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_x[2] = {tmem, tmem + 64}, t_y[2] = {tmem + 128, tmem + 192}, t_a1 = tmem + 256, t_a2 = tmem + 384;
    const bool bad = *abort_flag != 0;

    if (warp == 0 && !bad) {
        if (elect_one()) {
            mbar_expect_tx(bar(B_RES), 2 * T128);
            const int rr = row0 + tile * 128;
            if (IS_DQ) {
                tma_load_2d(s_r1, &tm_qkv128, head * D, rr, bar(B_RES));
                tma_load_2d(s_r1 + H128, &tm_qkv128, head * D + 64, rr, bar(B_RES));
                tma_load_2d(s_r2, &tm_do128, head * D, rr, bar(B_RES));
                tma_load_2d(s_r2 + H128, &tm_do128, head * D + 64, rr, bar(B_RES));
            } else {
                tma_load_2d(s_r1, &tm_qkv128, kcol, rr, bar(B_RES));
                tma_load_2d(s_r1 + H128, &tm_qkv128, kcol + 64, rr, bar(B_RES));
                tma_load_2d(s_r2, &tm_qkv128, vcol, rr, bar(B_RES));
                tma_load_2d(s_r2 + H128, &tm_qkv128, vcol + 64, rr, bar(B_RES));
            }
            for (int i = 0; i < n_items; ++i) {
                const int st = i % RING;
                if (!mbar_wait(bar(B_REMPTY + st), ((i / RING) & 1) ^ 1u, abort_flag)) break;
                mbar_expect_tx(bar(B_RFULL + st), STAGE);
                const uint32_t d1 = s_ring + st * STAGE, d2 = d1 + T64;
                if (IS_DQ) {
                    const int kr = row0 + (first_ct + i) * 64;
                    tma_load_2d(d1, &tm_qkv64, kcol, kr, bar(B_RFULL + st));
                    tma_load_2d(d1 + H64, &tm_qkv64, kcol + 64, kr, bar(B_RFULL + st));
                    tma_load_2d(d2, &tm_qkv64, vcol, kr, bar(B_RFULL + st));
                    tma_load_2d(d2 + H64, &tm_qkv64, vcol + 64, kr, bar(B_RFULL + st));
                } else {
                    const int h = hk * G + i / per_head, qr = row0 + (first_ct + i % per_head) * 64;
                    tma_load_2d(d1, &tm_qkv64, h * D, qr, bar(B_RFULL + st));
                    tma_load_2d(d1 + H64, &tm_qkv64, h * D + 64, qr, bar(B_RFULL + st));
                    tma_load_2d(d2, &tm_do64, h * D, qr, bar(B_RFULL + st));
                    tma_load_2d(d2 + H64, &tm_do64, h * D + 64, qr, bar(B_RFULL + st));
                }
            }
        }
    } else if (warp == 1 && !bad) {
        if (elect_one()) {
            const uint32_t idesc_s = make_idesc(1, 1, 0, 0, 128, 64), idesc_acc = make_idesc(1, 1, 0, 1, 128, 128);
            auto issue_acc = [&](int item) {
                const uint32_t c1 = s_ring + (item % RING) * STAGE, c2 = c1 + T64;
                if (IS_DQ) {
                    mma_acc_k64(t_a1, s_dst, c1, idesc_acc, item > 0);      // dQ += dS K
                } else {
                    mma_acc_k64(t_a1, s_pt, c2, idesc_acc, item > 0);       // dV += P^T dO
                    mma_acc_k64(t_a2, s_dst, c1, idesc_acc, item > 0);      // dK += dS^T Q
                }
                tc_commit(bar(B_REMPTY + item % RING));
                tc_commit(bar(B_PDSE));
            };
            bool ok = mbar_wait(bar(B_RES), 0, abort_flag);
            for (int i = 0; i < n_items && ok; ++i) {
                const int st = i % RING, xb = i & 1;
                if (!mbar_wait(bar(B_RFULL + st), (i / RING) & 1, abort_flag)) { ok = false; break; }
                if (!mbar_wait(bar(B_XYFREE + xb), ((i >> 1) & 1) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t c1 = s_ring + st * STAGE, c2 = c1 + T64;
                mma_128x64_kk(t_x[xb], s_r1, c1, idesc_s);     // S^T = K Q^T      |  S  = Q K^T
                mma_128x64_kk(t_y[xb], s_r2, c2, idesc_s);     // dP^T = V dO^T    |  dP = dO V^T
                tc_commit(bar(B_XY + xb));
                if (i >= 1) {
                    if (!mbar_wait(bar(B_PDS), (i - 1) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    issue_acc(i - 1);
                }
            }
            if (ok && n_items > 0 && mbar_wait(bar(B_PDS), (n_items - 1) & 1, abort_flag)) {
                tc_fence_after();
                issue_acc(n_items - 1);
                tc_commit(bar(B_DONE));
            }
        }
    } else if (warp >= 2 && !bad) {
        const int quad = warp & 3, r = quad * 32 + lane;
        const int half = (warp - 2) >> 2;                // which 32 of the item's 64 columns this warp handles
        const int t = (warp - 2) * 32 + lane;
        const int row_abs = tile * 128 + r;              // key position (dK/dV) or query position (dQ)
        const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
        float row_neg_lse2 = 0.f, row_dl = 0.f;
        int row_lo = 0;
        if (IS_DQ) {
            const size_t idx = static_cast<size_t>(row0 + row_abs) * p.Hq + head;
            row_neg_lse2 = -p.lse[idx] * LOG2E;
            row_dl = p.delta[idx];
            if (HAS_LO) row_lo = __ldg(p.lo + row0 + row_abs);
        }
        float pre_lse = 0.f, pre_dl = 0.f;
        int pre_lo = 0;
        if (!IS_DQ && t < 64 && n_items > 0) {
            const size_t idx = static_cast<size_t>(row0 + first_ct * 64 + t) * p.Hq + hk * G;
            pre_lse = p.lse[idx];
            pre_dl = p.delta[idx];
            if (HAS_LO) pre_lo = __ldg(p.lo + row0 + first_ct * 64 + t);
        }
        bool ok = true;
        const bool do_prof = p.prof != nullptr && threadIdx.x == 64 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
        long long acc_[6] = {0, 0, 0, 0, 0, 0};
        long long t_ = clock64();
        for (int i = 0; i < n_items && ok; ++i) {
            const int xb = i & 1;
            const int ct = first_ct + (IS_DQ ? i : i % per_head);     // index of the streamed 64-row tile inside the sequence
            const float* neg_lse2 = vec + xb * 128;
            const float* dl = neg_lse2 + 64;
            const int* q_lo = vec_lo + xb * 64;
            if (!IS_DQ) {
                if (t < 64) {        // values were fetched one item ahead (pre_lse / pre_dl), so their global-load latency is hidden
                    vec[xb * 128 + t] = -pre_lse * LOG2E;
                    vec[xb * 128 + 64 + t] = pre_dl;
                    if (HAS_LO) vec_lo[xb * 64 + t] = pre_lo;
                    if (i + 1 < n_items) {
                        const int h = hk * G + (i + 1) / per_head, nt = first_ct + (i + 1) % per_head;
                        const size_t idx = static_cast<size_t>(row0 + nt * 64 + t) * p.Hq + h;
                        pre_lse = p.lse[idx];
                        pre_dl = p.delta[idx];
                        if (HAS_LO) pre_lo = __ldg(p.lo + row0 + nt * 64 + t);
                    }
                }
                mbar_arrive(bar(B_VEC));
                if (!mbar_wait(bar(B_VEC), i & 1, abort_flag)) { ok = false; break; }
            }
            FB_PROF(0);
            if (!mbar_wait(bar(B_XY + xb), (i >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            FB_PROF(1);
            float x[32], y[32];
            ld32f(t_x[xb] + lane_sel + half * 32, x);
            ld32f(t_y[xb] + lane_sel + half * 32, y);
            tc_fence_before();
            mbar_arrive(bar(B_XYFREE + xb));
            FB_PROF(2);
            const int c0 = ct * 64 + half * 32;
            // causal mask: a key may not be later than the query.  dK/dV: row = key, column = query; dQ: row = query, column = key.
            const bool diag = IS_DQ ? (ct >= 2 * tile) : (ct < 2 * tile + 2);
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                float pr = ex2_approx(fmaf(x[c], p.scale_log2, IS_DQ ? row_neg_lse2 : neg_lse2[half * 32 + c]));
                if (diag && (IS_DQ ? (c0 + c > row_abs) : (row_abs > c0 + c))) pr = 0.f;
                // lower bound: a key before the query's first visible key contributes nothing
                if (HAS_LO && (IS_DQ ? (c0 + c < row_lo) : (row_abs < q_lo[half * 32 + c]))) pr = 0.f;
                x[c] = pr;
                y[c] = pr * (y[c] - (IS_DQ ? row_dl : dl[half * 32 + c])) * p.scale;
            }
            FB_PROF(3);
            if (i > 0 && !mbar_wait(bar(B_PDSE), (i - 1) & 1, abort_flag)) { ok = false; break; }
            FB_PROF(4);
            if (!IS_DQ) store_row32h(pt_tile, r, half, x);
            store_row32h(dst_tile, r, half, y);
            fence_proxy_async();
            mbar_arrive(bar(B_PDS));
            FB_PROF(5);
        }
        if (do_prof) {
            long long* dst = p.prof + (IS_DQ ? 8 : 0);
            for (int k = 0; k < 6; ++k) dst[k] = acc_[k];
            dst[6] = n_items;
        }
        if (ok && n_items > 0 && mbar_wait(bar(B_DONE), 0, abort_flag)) {
            tc_fence_after();
            const size_t width = static_cast<size_t>(p.Hq + 2 * p.Hkv) * D;
            __nv_bfloat16* base = p.d_qkv + static_cast<size_t>(row0 + row_abs) * width;
            if (IS_DQ) {
                store_acc128(t_a1, lane_sel, base + head * D, half);
            } else {
                store_acc128(t_a2, lane_sel, base + kcol, half);
                store_acc128(t_a1, lane_sel, base + vcol, half);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.error_flag) atomicExch(p.error_flag, IS_DQ ? 8 : 9);
    if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

}  // namespace fb64

const char* flash_attn_bwd64_sm100(const void* qkv, const void* d_out, const float* lse, const float* delta, void* d_qkv, int B, int T, int Hq, int Hkv,
                                   float softmax_scale, int* error_flag, cudaStream_t stream, long long* prof, const int* lo, const int* kv_qend) {
    using namespace fb64;
    if (T % 128 != 0) return "flash_attn_bwd: T must be a multiple of 128";
    CUtensorMap q128, q64, do128, do64;
    const uint64_t width = static_cast<uint64_t>(Hq + 2 * Hkv) * D, owidth = static_cast<uint64_t>(Hq) * D, rows = static_cast<uint64_t>(B) * T;
    const char* e = nullptr;
    if ((e = make_tensor_map_2d(&q128, qkv, 2, width, rows, width * 2, 64, 128))) return e;
    if ((e = make_tensor_map_2d(&q64, qkv, 2, width, rows, width * 2, 64, 64))) return e;
    if ((e = make_tensor_map_2d(&do128, d_out, 2, owidth, rows, owidth * 2, 64, 128))) return e;
    if ((e = make_tensor_map_2d(&do64, d_out, 2, owidth, rows, owidth * 2, 64, 64))) return e;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(fa_bwd64_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(fa_bwd64_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(fa_bwd64_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(fa_bwd64_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return "cudaFuncSetAttribute failed (flash_attn_bwd64)";
        attr_set = true;
    }
    if ((lo == nullptr) != (kv_qend == nullptr)) return "flash_attn_bwd: the lower bounds and the per-key-tile query ends come together";
    Params p{static_cast<__nv_bfloat16*>(d_qkv), lse, delta, T, Hq, Hkv, softmax_scale, softmax_scale * LOG2E, error_flag, prof, lo, kv_qend};
    if (lo) {
        fa_bwd64_kernel<false, true><<<dim3(T / 128, Hkv, B), THREADS, SMEM, stream>>>(q128, q64, do128, do64, p);
        fa_bwd64_kernel<true, true><<<dim3(T / 128, Hq, B), THREADS, SMEM, stream>>>(q128, q64, do128, do64, p);
    } else {
        fa_bwd64_kernel<false, false><<<dim3(T / 128, Hkv, B), THREADS, SMEM, stream>>>(q128, q64, do128, do64, p);
        fa_bwd64_kernel<true, false><<<dim3(T / 128, Hq, B), THREADS, SMEM, stream>>>(q128, q64, do128, do64, p);
    }
    return cudaGetLastError() == cudaSuccess ? nullptr : "flash_attn_bwd64 launch failed";
}

// delta[b, t, h] = sum_d dO * O   (one warp per (token, head))
__global__ void __launch_bounds__(256) fa_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                                                       size_t items) {
    const int lane = threadIdx.x & 31;
    for (size_t it = blockIdx.x * static_cast<size_t>(blockDim.x >> 5) + (threadIdx.x >> 5); it < items; it += static_cast<size_t>(gridDim.x) * (blockDim.x >> 5)) {
        const uint2 a = *reinterpret_cast<const uint2*>(o + it * 128 + lane * 4), g = *reinterpret_cast<const uint2*>(d_o + it * 128 + lane * 4);
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

const char* flash_attn_bwd_sm100(const void* qkv, const void* out, const void* d_out, const float* lse, float* delta, void* d_qkv, int B, int T, int Hq,
                                 int Hkv, float softmax_scale, int* error_flag, int num_sms, cudaStream_t stream, const int* lo, const int* kv_qend) {
    if (T % 128 != 0) return "flash_attn_bwd: T must be a multiple of 128";
    const size_t items = static_cast<size_t>(B) * T * Hq;
    int grid = static_cast<int>((items + 7) / 8);
    if (grid > num_sms * 8) grid = num_sms * 8;
    fa_delta_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(d_out), delta, items);
    return flash_attn_bwd64_sm100(qkv, d_out, lse, delta, d_qkv, B, T, Hq, Hkv, softmax_scale, error_flag, stream, nullptr, lo, kv_qend);
}

}  // namespace sg

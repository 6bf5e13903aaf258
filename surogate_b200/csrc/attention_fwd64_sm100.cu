// Flash-attention forward, second generation: 128 queries x 64 keys per step, sized so that TWO CTAs fit on one SM
// (112 KB shared memory and 256 TMEM columns each).  While one CTA's softmax warps work on their scores, the other CTA's
// MMAs keep the tensor core busy; the same overlap a two-tile ping-pong gives, obtained from the hardware scheduler.
// Causal, GQA, head_dim 128, packed QKV [B, T, (Hq + 2 Hkv) * 128] read by TMA.
//   warp 0      TMA producer: Q once, then K_j / V_j tiles through two 2-deep rings
//   warp 1      MMA issuer:   S_j = Q K_j^T into one of two TMEM score buffers, then O += P_j V_j (V read MN-major)
//   warps 2-5   softmax:      thread r owns query row r: reads S_j from TMEM, online softmax in base 2, writes P_j (bf16) to shared
//                             memory in the swizzled K-major layout the second MMA reads; the running output in TMEM is rescaled
//                             only when a row maximum grew by more than 2^8 (exact, but rare)
// Optional per-row LOWER BOUND `lo[b, t]` (HAS_LO): query t attends keys lo[t] <= k <= t.  One array covers packed documents
// (lo = first position of the query's document), sliding windows (lo = t - window + 1) and both at once (the maximum).  `lo` must be
// non-decreasing along a sequence, so a query tile starts at key tile lo[first row] / 64 and key tiles before it are never loaded.
// Replaces the varlen FlashAttention call of the reference (csrc/src/runtime/attention/backend_flash_varlen.cpp:41-63).
#include <cuda_bf16.h>
#include <math_constants.h>

#include "attention_sm100.h"
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace sg {
namespace fa64 {

constexpr int BQ = 128, BKV = 64, D = 128;
constexpr int Q_BYTES = BQ * D * 2;          // 32 KB: two halves (d 0..63, 64..127) of 128 rows x 128 B
constexpr int Q_HALF = 16384;
constexpr int KV_TILE = BKV * D * 2;         // 16 KB: two halves of 64 rows x 128 B
constexpr int KV_HALF = 8192;
constexpr int P_BYTES = BQ * BKV * 2;        // 16 KB: 128 rows x 128 B
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 256;               // S0 [0,64) S1 [64,128) O [128,256)
constexpr float RESCALE_THRESHOLD = 8.f;
// layout: Q | K0 V0 | K1 V1 | P | barriers + flags
constexpr int OFF_KV = Q_BYTES, OFF_P = OFF_KV + 4 * KV_TILE, OFF_BAR = OFF_P + P_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 256;

struct Params {
    __nv_bfloat16* out;
    float* lse;
    int T, Hq, Hkv;
    float scale_log2;
    int* error_flag;
    long long* prof;      // optional [8] cycle counters of one softmax thread (development aid; nullptr in production)
    const int* lo;        // optional [B, T] first key each query may attend (position inside its sequence)
};

#define FA_PROF(k)                                   \
    do {                                             \
        if (do_prof) {                               \
            const long long now_ = clock64();        \
            acc_[k] += now_ - t_;                    \
            t_ = now_;                               \
        }                                            \
    } while (0)

template <bool HAS_LO>
__global__ void __launch_bounds__(THREADS, 2) fa_fwd64_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                                                              const Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t s0 = smem_u32(smem);
    const uint32_t s_q = s0, s_kv = s0 + OFF_KV, s_p = s0 + OFF_P, bars = s0 + OFF_BAR;
    uint8_t* p_tile = smem + OFF_P;
    // barriers: 0 q_full | 1,2 k_full | 3,4 k_empty | 5,6 s_full | 7,8 s_empty | 9 p_full | 10 p_empty | 11 o_full | 12,13 v_full | 14,15 v_empty
    // K and V travel through separate 2-deep rings: a K slot is free as soon as S_j has been computed, so K_{j+2} is requested two
    // steps ahead of its use, and V_{j+2} as soon as P_j V_j is done (V is needed later in a step than K).
    auto bar = [&](int i) { return bars + 8u * i; };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_BAR + 136);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_blk = gridDim.x - 1 - blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.Hq / p.Hkv);
    const int row0 = b * p.T;
    // key tiles [j0, j0 + n_kv) are visited; without a lower bound that is everything up to the diagonal
    const int j0 = HAS_LO ? __ldg(p.lo + row0 + q_blk * BQ) / BKV : 0;
    const int n_kv = 2 * (q_blk + 1) - j0;

    if (threadIdx.x == 0) {
        *abort_flag = (s0 & 1023u) ? 1 : 0;      // the swizzled tiles need a 1024-byte aligned base
        mbar_init(bar(0), 1);
        for (int i = 1; i <= 8; ++i) mbar_init(bar(i), (i == 7 || i == 8) ? 128 : 1);
        mbar_init(bar(9), 128);
        mbar_init(bar(10), 1);
        mbar_init(bar(11), 1);
        for (int i = 12; i <= 15; ++i) mbar_init(bar(i), 1);
        fence_barrier_init();
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_kv);
    }
    if (warp == 2) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_s[2] = {tmem, tmem + 64}, t_o = tmem + 128;
    const bool bad = *abort_flag != 0;

    if (warp == 0 && !bad) {
        if (elect_one()) {
            mbar_expect_tx(bar(0), Q_BYTES);
            tma_load_2d(s_q, &tm_q, h * D, row0 + q_blk * BQ, bar(0));
            tma_load_2d(s_q + Q_HALF, &tm_q, h * D + 64, row0 + q_blk * BQ, bar(0));
            const int kc = (p.Hq + hk) * D, vc = (p.Hq + p.Hkv + hk) * D;
            // K_j is requested one step ahead of V_{j-1}: a late V slot must not hold back the next K request
            for (int j = 0; j <= n_kv; ++j) {
                if (j < n_kv) {
                    const int st = j & 1;
                    if (!mbar_wait(bar(3 + st), ((j >> 1) & 1) ^ 1u, abort_flag)) break;
                    const uint32_t k_dst = s_kv + st * 2 * KV_TILE;
                    mbar_expect_tx(bar(1 + st), KV_TILE);
                    tma_load_2d(k_dst, &tm_kv, kc, row0 + (j0 + j) * BKV, bar(1 + st));
                    tma_load_2d(k_dst + KV_HALF, &tm_kv, kc + 64, row0 + (j0 + j) * BKV, bar(1 + st));
                }
                if (j >= 1) {
                    const int i = j - 1, st = i & 1;
                    if (!mbar_wait(bar(14 + st), ((i >> 1) & 1) ^ 1u, abort_flag)) break;
                    const uint32_t v_dst = s_kv + st * 2 * KV_TILE + KV_TILE;
                    mbar_expect_tx(bar(12 + st), KV_TILE);
                    tma_load_2d(v_dst, &tm_kv, vc, row0 + (j0 + i) * BKV, bar(12 + st));
                    tma_load_2d(v_dst + KV_HALF, &tm_kv, vc + 64, row0 + (j0 + i) * BKV, bar(12 + st));
                }
            }
        }
    } else if (warp == 1 && !bad) {
        if (elect_one()) {
            const uint32_t idesc_s = make_idesc(1, 1, 0, 0, 128, 64);      // S[128 q, 64 keys]
            const uint32_t idesc_pv = make_idesc(1, 1, 0, 1, 128, 128);    // O[128 q, 128 d], V read MN-major
            // S = Q K^T: contraction d = 128 = 2 halves x 4 steps of 16
            auto issue_s = [&](uint32_t d_tmem, uint32_t k_base) {
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        mma_f16(d_tmem, make_smem_desc(s_q + c * Q_HALF + ks * 32, 16, 1024), make_smem_desc(k_base + c * KV_HALF + ks * 32, 16, 1024),
                                idesc_s, (c > 0 || ks > 0) ? 1u : 0u);
            };
            // O += P V: contraction = 64 keys = 4 steps of 16; V halves (d chunks) are KV_HALF apart
            auto issue_pv = [&](uint32_t v_base, bool acc) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    mma_f16(t_o, make_smem_desc(s_p + ks * 32, 16, 1024), make_smem_desc(v_base + ks * 2048, KV_HALF, 1024), idesc_pv,
                            (acc || ks > 0) ? 1u : 0u);
            };
            bool ok = mbar_wait(bar(0), 0, abort_flag);
            for (int j = 0; j < n_kv && ok; ++j) {
                const int st = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                if (!mbar_wait(bar(1 + st), ph, abort_flag)) { ok = false; break; }
                if (!mbar_wait(bar(7 + st), ph ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                issue_s(t_s[st], s_kv + st * 2 * KV_TILE);
                tc_commit(bar(5 + st));
                tc_commit(bar(3 + st));                     // K slot reusable once S_j is computed
                if (j >= 1) {
                    const int pst = (j - 1) & 1;
                    if (!mbar_wait(bar(12 + pst), ((j - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                    if (!mbar_wait(bar(9), (j - 1) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    issue_pv(s_kv + pst * 2 * KV_TILE + KV_TILE, j - 1 > 0);
                    tc_commit(bar(14 + pst));
                    tc_commit(bar(10));
                }
            }
            if (ok && mbar_wait(bar(12 + ((n_kv - 1) & 1)), ((n_kv - 1) >> 1) & 1, abort_flag) && mbar_wait(bar(9), (n_kv - 1) & 1, abort_flag)) {
                tc_fence_after();
                const int pst = (n_kv - 1) & 1;
                issue_pv(s_kv + pst * 2 * KV_TILE + KV_TILE, n_kv - 1 > 0);
                tc_commit(bar(14 + pst));
                tc_commit(bar(10));
                tc_commit(bar(11));
            }
        }
    } else if (warp >= 2 && !bad) {
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const int q_abs = q_blk * BQ + r;            // query position inside the sequence
        const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
        // a finite floor instead of -inf: a row whose first visited key tile is entirely masked keeps exp2(s - m) = 0 instead of NaN
        float m_used = -1e30f, l = 0.f;
        const int lo_row = HAS_LO ? __ldg(p.lo + row0 + q_abs) : 0;
        bool ok = true;
        const bool do_prof = p.prof != nullptr && threadIdx.x == 64 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
        long long acc_[6] = {0, 0, 0, 0, 0, 0};
        long long t_ = clock64();
        for (int j = 0; j < n_kv && ok; ++j) {
            const int st = j & 1;
            if (!mbar_wait(bar(5 + st), (j >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            FA_PROF(0);
            float s[64];                                // raw (unscaled) scores; the softmax scale is folded into one FMA below
            {
                uint32_t ra[32], rb[32];
                tmem_ld_32x32(t_s[st] + lane_sel, ra);
                tmem_ld_32x32(t_s[st] + lane_sel + 32, rb);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) { s[i] = __uint_as_float(ra[i]); s[32 + i] = __uint_as_float(rb[i]); }
            }
            tc_fence_before();
            mbar_arrive(bar(7 + st));
            FA_PROF(1);
            const int k0 = (j0 + j) * BKV;
            if (j0 + j >= 2 * q_blk) {                 // the two key tiles that straddle the diagonal
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (k0 + i > q_abs) s[i] = -CUDART_INF_F;
            }
            if (HAS_LO && k0 < lo_row) {               // keys before the row's lower bound (another document / outside the window)
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (k0 + i < lo_row) s[i] = -CUDART_INF_F;
            }
            // four independent chains instead of one 64-long dependent chain (one warp per scheduler has no other work to hide latency)
            float m4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
            for (int i = 4; i < 64; ++i) m4[i & 3] = fmaxf(m4[i & 3], s[i]);
            const float m_blk = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
            // a fully masked row (second diagonal tile, upper half of the rows; tiles before the row's lower bound) has m_blk = -inf:
            // nothing to add, keep m_used
            const bool grow = m_blk > m_used + RESCALE_THRESHOLD;
            FA_PROF(2);
            if (j > 0) {
                if (!mbar_wait(bar(10), (j - 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                FA_PROF(3);
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
            const float neg_m = -m_used;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint8_t* prow = p_tile + r * 128;
#pragma unroll
            for (int u = 0; u < 8; ++u) {              // 8 units of 8 keys (16 bytes), swizzled by the row index
                uint4 o;
                __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float a = ex2_approx(fmaf(s[u * 8 + 2 * i], p.scale_log2, neg_m));
                    const float c = ex2_approx(fmaf(s[u * 8 + 2 * i + 1], p.scale_log2, neg_m));
                    sum4[i] += a + c;
                    po[i] = __floats2bfloat162_rn(a, c);
                }
                *reinterpret_cast<uint4*>(prow + ((u ^ (r & 7)) << 4)) = o;
            }
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            l += sum;
            FA_PROF(4);
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(bar(9));
            FA_PROF(5);
        }
        if (do_prof) {
            for (int k = 0; k < 6; ++k) p.prof[k] = acc_[k];
            p.prof[6] = n_kv;
        }
        if (ok && mbar_wait(bar(11), 0, abort_flag)) {
            tc_fence_after();
            const float inv = 1.f / l;
            __nv_bfloat16* orow = p.out + (static_cast<size_t>(row0 + q_abs) * p.Hq + h) * D;
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
            p.lse[static_cast<size_t>(row0 + q_abs) * p.Hq + h] = (m_used + log2f(l)) * 0.6931471805599453f;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.error_flag) atomicExch(p.error_flag, 7);
    if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

}  // namespace fa64

const char* flash_attn_fwd64_sm100(const void* qkv, void* out, float* lse, int B, int T, int Hq, int Hkv, float softmax_scale, int* error_flag,
                                   cudaStream_t stream, long long* prof, const int* lo) {
    using namespace fa64;
    if (T % 128 != 0) return "flash_attn_fwd: T must be a multiple of 128";
    if (Hq % Hkv != 0) return "flash_attn_fwd: Hq must be a multiple of Hkv";
    CUtensorMap tm_q, tm_kv;
    const uint64_t width = static_cast<uint64_t>(Hq + 2 * Hkv) * D;
    const char* e = make_tensor_map_2d(&tm_q, qkv, 2, width, static_cast<uint64_t>(B) * T, width * 2, 64, 128);
    if (e) return e;
    e = make_tensor_map_2d(&tm_kv, qkv, 2, width, static_cast<uint64_t>(B) * T, width * 2, 64, 64);
    if (e) return e;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(fa_fwd64_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(fa_fwd64_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
            return "cudaFuncSetAttribute failed (flash_attn_fwd64)";
        attr_set = true;
    }
    Params p{static_cast<__nv_bfloat16*>(out), lse, T, Hq, Hkv, softmax_scale * 1.4426950408889634f, error_flag, prof, lo};
    if (lo) fa_fwd64_kernel<true><<<dim3(T / 128, Hq, B), THREADS, SMEM_BYTES, stream>>>(tm_q, tm_kv, p);
    else fa_fwd64_kernel<false><<<dim3(T / 128, Hq, B), THREADS, SMEM_BYTES, stream>>>(tm_q, tm_kv, p);
    return cudaGetLastError() == cudaSuccess ? nullptr : "flash_attn_fwd64 launch failed";
}

}  // namespace sg

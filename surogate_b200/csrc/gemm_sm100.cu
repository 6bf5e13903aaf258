// Dense GEMM for sm_100a: D[M,N] = alpha * sa * sb * (A[M,K] . B[N,K]^T) (+ D), fp32 accumulation in TMEM.
//
// * Inputs bf16 (tcgen05 kind::f16) or FP8 e4m3/e5m2 in any mix (kind::f8f6f4).
// * Each operand may be K-major ([rows, K] row-major) or MN-major ([K, rows] row-major).  Forward (x.W^T),
//   dgrad (dy.W) and wgrad (dy^T.x) therefore all read the tensors as they lie in memory: no transposed
//   copies of weights or activations are ever made, for bf16 or FP8.
// * Persistent, warp-specialised: warp 0 issues TMA loads into a multi-stage shared-memory ring, warp 1
//   issues tcgen05.mma (one elected thread), warps 2-5 drain the accumulator from TMEM (tcgen05.ld), apply
//   the scales and write bf16 / fp32.  Two accumulators (2 x BN TMEM columns) let the epilogue of tile i
//   overlap the main loop of tile i+1.
// * Optional epilogue extras: accumulate into D (gradient accumulation), running abs-max of the output.
// * No cluster multicast anywhere (loads are per-CTA), so the same kernel is used at any GPU count.
//
// Replaces the cuBLASLt calls of the reference (csrc/src/kernels/matmul.cpp:447-1000).
#include <cuda_fp8.h>

#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace sg {

constexpr int BM = 128;
constexpr int TILE_K_BYTES = 128;   // one swizzle row
constexpr int A_STAGE_BYTES = BM * TILE_K_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 8;

template <int BN> struct Cfg {
    static constexpr int B_STAGE_BYTES = BN * TILE_K_BYTES;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr int STAGES = (BN == 256) ? 4 : 6;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
    static constexpr int TMEM_COLS = 2 * BN;
};

// What one output tile needs to know.  Coordinates are TMA coordinates (elements).
struct TileInfo {
    int a_row0;   // A: row (K-major) or M-column (MN-major) coordinate of the tile
    int b_row0;   // B: row (K-major) or N-column (MN-major) coordinate of the tile
    int a_k0;     // first contraction coordinate in A
    int b_k0;     // first contraction coordinate in B
    int num_k;    // contraction blocks
    int d_row0, d_col0;   // output tile origin
    int m_end, n_end;     // exclusive store limits
    long long d_off;      // element offset of this tile's output matrix inside D
};

// Tile schedules.  mode 0: one dense problem.  mode 1: rows of A / D are grouped (MoE forward and dgrad): group g owns rows
// [offs[g], offs[g+1]) (multiples of 128) and uses B block g.  mode 2: the contraction is grouped (MoE wgrad): group g
// contracts rows [offs[g], offs[g+1]) of both operands into output matrix g.
__device__ __forceinline__ int find_group(const int* tile_start, int num_groups, int tile) {
    int lo = 0, hi = num_groups;  // largest g with tile_start[g] <= tile
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tile_start[mid] <= tile) lo = mid; else hi = mid;
    }
    return lo;
}

template <int BN>
__device__ __forceinline__ TileInfo get_tile(const GemmParams& p, const int* tile_start, int tile, int BK) {
    TileInfo t;
    const int num_n = (p.N + BN - 1) / BN;
    if (p.mode == 0) {
        const int num_m = (p.M + BM - 1) / BM;
        const int per_group = GROUP_M * num_n;
        const int group = tile / per_group;
        const int first_m = group * GROUP_M;
        const int gsize = min(num_m - first_m, GROUP_M);
        const int r = tile - group * per_group;
        const int m_blk = first_m + r % gsize, n_blk = r / gsize;
        t.a_row0 = t.d_row0 = m_blk * BM;
        t.b_row0 = t.d_col0 = n_blk * BN;
        t.a_k0 = t.b_k0 = 0;
        t.num_k = (p.K + BK - 1) / BK;
        t.m_end = p.M;
        t.n_end = p.N;
        t.d_off = 0;
    } else if (p.mode == 1) {
        const int g = find_group(tile_start, p.num_groups, tile);
        const int local = tile - tile_start[g];
        const int m_tiles = (p.group_offsets[g + 1] - p.group_offsets[g]) / BM;
        const int m_blk = local % m_tiles, n_blk = local / m_tiles;
        t.a_row0 = t.d_row0 = p.group_offsets[g] + m_blk * BM;
        t.d_col0 = n_blk * BN;
        // B block g: K-major weights are stacked on rows ([G*N, K]); MN-major weights are stacked on the contraction ([G*K, N])
        t.b_row0 = p.b_mn ? n_blk * BN : g * p.N + n_blk * BN;
        t.a_k0 = 0;
        t.b_k0 = p.b_mn ? g * p.K : 0;
        t.num_k = (p.K + BK - 1) / BK;
        t.m_end = p.group_offsets[g + 1];
        t.n_end = p.N;
        t.d_off = 0;
    } else {
        const int num_m = (p.M + BM - 1) / BM;
        const int per = num_m * num_n;
        const int g = find_group(tile_start, p.num_groups, tile);
        const int local = tile - tile_start[g];
        const int m_blk = local % num_m, n_blk = local / num_m;
        t.a_row0 = t.d_row0 = m_blk * BM;
        t.b_row0 = t.d_col0 = n_blk * BN;
        t.a_k0 = t.b_k0 = p.group_offsets[g];
        t.num_k = (p.group_offsets[g + 1] - p.group_offsets[g]) / BK;
        t.m_end = p.M;
        t.n_end = p.N;
        t.d_off = static_cast<long long>(g) * p.M * p.N;
        (void)per;
    }
    return t;
}

// 32 accumulator columns of one output row, straight from registers: 16-byte stores, optional D += and running abs-max.
__device__ __forceinline__ void store_direct_32(const GemmParams& p, const TileInfo& t, int row, int col0, const uint32_t (&r)[32], float scale,
                                                float& amax) {
    if (row >= t.m_end || col0 >= t.n_end) return;
    if (p.out_fp32) {
        float* drow = reinterpret_cast<float*>(p.D) + t.d_off + static_cast<size_t>(row) * p.ldd + col0;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            if (col0 + g * 4 < t.n_end) {
                float4 v = make_float4(__uint_as_float(r[g * 4]) * scale, __uint_as_float(r[g * 4 + 1]) * scale, __uint_as_float(r[g * 4 + 2]) * scale,
                                       __uint_as_float(r[g * 4 + 3]) * scale);
                float4* dst = reinterpret_cast<float4*>(drow + g * 4);
                if (p.accumulate) {
                    const float4 o = *dst;
                    v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                *dst = v;
            }
        }
    } else {
        __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.D) + t.d_off + static_cast<size_t>(row) * p.ldd + col0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            if (col0 + g * 8 < t.n_end) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]) * scale;
                uint4* dst = reinterpret_cast<uint4*>(drow + g * 8);
                if (p.accumulate) {
                    const uint4 o = *dst;
                    const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __bfloat1622float2(ob[i]);
                        v[2 * i] += f.x;
                        v[2 * i + 1] += f.y;
                    }
                }
                uint4 out;
                __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    pb[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                    amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
                }
                *dst = out;
            }
        }
    }
}

constexpr int MAX_GROUPS = 256;

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + C::STAGES * C::STAGE_BYTES;
    // barrier layout (8 B each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * C::STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * C::STAGES + 2 + a); };
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int elems_per_row = TILE_K_BYTES / p.elem_bytes;  // K elements per stage (K-major) = BK
    const int BK = elems_per_row;
    __shared__ int tile_start[MAX_GROUPS + 1];
    __shared__ int num_tiles_sh;
    if (p.mode == 0) {
        if (threadIdx.x == 0) num_tiles_sh = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
    } else if (threadIdx.x == 0) {
        // prefix of tiles per group (<= 256 groups: a serial scan by one thread costs well under a microsecond)
        const int num_n = (p.N + BN - 1) / BN;
        int acc = 0;
        for (int g = 0; g < p.num_groups; ++g) {
            tile_start[g] = acc;
            const int rows = p.group_offsets[g + 1] - p.group_offsets[g];
            if (p.mode == 1) acc += (rows / BM) * num_n;
            else acc += rows > 0 ? ((p.M + BM - 1) / BM) * num_n : 0;   // empty groups contribute no tiles
        }
        tile_start[p.num_groups] = acc;
        num_tiles_sh = acc;
    }

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 128);
        }
        fence_barrier_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 2) {
        tmem_alloc(smem_u32(&tmem_base_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const int num_tiles = num_tiles_sh;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            const int a_chunks = p.a_mn ? (BM * p.elem_bytes) / TILE_K_BYTES : 1;
            const int b_chunks = p.b_mn ? (BN * p.elem_bytes) / TILE_K_BYTES : 1;
            const int chunk_bytes = BK * TILE_K_BYTES;   // MN-major chunk: BK rows of 128 B
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const TileInfo t = get_tile<BN>(p, tile_start, tile, BK);
                const int m0 = t.a_row0, n0 = t.b_row0;
                for (int kb = 0; kb < t.num_k; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, &abort_flag)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * C::STAGE_BYTES;
                    const uint32_t sb = sa + A_STAGE_BYTES;
                    mbar_expect_tx(full_bar(stage), C::STAGE_BYTES);
                    const int ka = t.a_k0 + kb * BK, kbb = t.b_k0 + kb * BK;
                    if (!p.a_mn) {
                        tma_load_2d(sa, &tmA, ka, m0, full_bar(stage));
                    } else {
                        for (int c = 0; c < a_chunks; ++c) tma_load_2d(sa + c * chunk_bytes, &tmA, m0 + c * elems_per_row, ka, full_bar(stage));
                    }
                    if (!p.b_mn) {
                        tma_load_2d(sb, &tmB, kbb, n0, full_bar(stage));
                    } else {
                        for (int c = 0; c < b_chunks; ++c) tma_load_2d(sb + c * chunk_bytes, &tmB, n0 + c * elems_per_row, kbb, full_bar(stage));
                    }
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t acc_phase[2] = {0, 0};
            int local_tile = 0;
            const uint32_t idesc = make_idesc(p.a_fmt, p.b_fmt, p.a_mn, p.b_mn, BM, BN);
            const uint32_t lbo = BK * TILE_K_BYTES;                 // MN-major: stride between 128-byte MN chunks
            const uint32_t a_kstep = p.a_mn ? (BK / 4) * TILE_K_BYTES : 32;
            const uint32_t b_kstep = p.b_mn ? (BK / 4) * TILE_K_BYTES : 32;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
                const int acc = local_tile & 1;
                if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, &abort_flag)) { ok = false; break; }
                acc_phase[acc] ^= 1u;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                const int num_k = get_tile<BN>(p, tile_start, tile, BK).num_k;
                for (int kb = 0; kb < num_k; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, &abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_base + stage * C::STAGE_BYTES;
                    const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t da = make_smem_desc(sa + j * a_kstep, p.a_mn ? lbo : 16, 1024);
                        const uint64_t db = make_smem_desc(sb + j * b_kstep, p.b_mn ? lbo : 16, 1024);
                        const uint32_t accum = (kb > 0 || j > 0) ? 1u : 0u;
                        if (p.elem_bytes == 2) mma_f16(d_tmem, da, db, idesc, accum);
                        else mma_f8(d_tmem, da, db, idesc, accum);
                    }
                    tc_commit(empty_bar(stage));   // frees the smem stage once these MMAs have read it
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) tc_commit(tfull_bar(acc));   // accumulator complete
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quad = warp & 3;          // TMEM lane quarter this warp may access
        uint32_t acc_phase[2] = {0, 0};
        int local_tile = 0;
        float scale = p.alpha;
        if (p.scale_a) scale *= __ldg(p.scale_a);
        if (p.scale_b) scale *= __ldg(p.scale_b);
        float amax = 0.f;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
            const TileInfo t = get_tile<BN>(p, tile_start, tile, BK);
            const int acc = local_tile & 1;
            if (!mbar_wait(tfull_bar(acc), acc_phase[acc], &abort_flag)) { ok = false; break; }
            acc_phase[acc] ^= 1u;
            tc_fence_after();
            const int row = t.d_row0 + quad * 32 + lane;
            const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld_32x32(t_row + c, r);
                tmem_ld_wait();
                store_direct_32(p, t, row, t.d_col0 + c, r, scale, amax);
            }
            tc_fence_before();
            mbar_arrive(tempty_bar(acc));
        }
        if (p.amax_out) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (lane == 0 && amax > 0.f) atomicMax(reinterpret_cast<unsigned int*>(p.amax_out), __float_as_uint(amax));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag && p.error_flag) atomicExch(p.error_flag, 1);
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------ CTA-pair kernel
// 256 x 256 output tile per CLUSTER of two CTAs (tcgen05 cta_group::2).  Each CTA stages its own 128 rows of A and its own 128 of
// the tile's 256 B rows (16 KB + 16 KB per stage instead of 16 + 32 for the single-CTA 128 x 256 tile, so six stages fit and every
// byte of B is read from shared memory by one SM, not two); the leader CTA's MMA thread issues M = 256, N = 256 instructions that
// fill 128 TMEM lanes x 256 columns in both CTAs.  Loads are per-CTA TMA copies (no cluster broadcast) that complete on the
// leader's barrier; the MMA completion is committed to both CTAs' barriers.  The epilogue leaves through shared memory: every
// warp packs its 32 rows x 128 bytes into a swizzled staging tile and one lane issues a TMA store (or a TMA add for fp32
// accumulation), so global writes are whole 128-byte lines and the tensor map clips the edges.  bf16 accumulation and the
// running abs-max of accumulated outputs keep the register path.  Dense problems only (mode 0).
constexpr int PAIR_BM = 256, PAIR_BN = 256;
constexpr int PAIR_B_BYTES = 128 * TILE_K_BYTES;                 // this CTA's half of the B tile
constexpr int PAIR_STAGE_BYTES = A_STAGE_BYTES + PAIR_B_BYTES;   // 32 KB
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_EPI_WARP_BYTES = 2 * 4096;                    // two 32-row x 128-byte staging tiles per epilogue warp
constexpr int PAIR_EPI_BYTES = 4 * PAIR_EPI_WARP_BYTES;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + PAIR_EPI_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

struct PairTile {
    int m0, n0;   // origin of the 256 x 256 tile
};
__device__ __forceinline__ PairTile pair_tile(const GemmParams& p, int tile) {
    const int num_m = (p.M + PAIR_BM - 1) / PAIR_BM, num_n = (p.N + PAIR_BN - 1) / PAIR_BN;
    const int per_group = p.pair_group_m * num_n;
    const int group = tile / per_group;
    const int first_m = group * p.pair_group_m;
    const int gsize = min(num_m - first_m, p.pair_group_m);
    const int r = tile - group * per_group;
    return PairTile{(first_m + r % gsize) * PAIR_BM, (r / gsize) * PAIR_BN};
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmD,
                 const GemmParams p, const int use_tma_store) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // same offset in both CTAs: the MMA applies one descriptor to both
    const uint32_t epi_base = smem_base + PAIR_STAGES * PAIR_STAGE_BYTES;
    const uint32_t bar_base = epi_base + PAIR_EPI_BYTES;
    // barriers (8 B each): full[STAGES] (used in the leader), empty[STAGES], tmem_full[2], tmem_empty[2] (used in the leader)
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (PAIR_STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * PAIR_STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * PAIR_STAGES + 2 + a); };
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int BK = TILE_K_BYTES / p.elem_bytes;
    const int num_tiles = ((p.M + PAIR_BM - 1) / PAIR_BM) * ((p.N + PAIR_BN - 1) / PAIR_BN);
    const int num_k = (p.K + BK - 1) / BK;
    const int first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);      // one lane of each epilogue warp of both CTAs
        }
        fence_barrier_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if (use_tma_store) tma_prefetch_desc(&tmD);
    }
    if (warp == 2) {
        tmem_alloc_pair(smem_u32(&tmem_base_slot), 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    cluster_sync_all();     // both CTAs' barriers are initialised before either CTA signals the other
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (one per CTA)
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            const int a_chunks = p.a_mn ? (BM * p.elem_bytes) / TILE_K_BYTES : 1;
            const int b_chunks = p.b_mn ? (128 * p.elem_bytes) / TILE_K_BYTES : 1;
            const int chunk_bytes = BK * TILE_K_BYTES;
            bool ok = true;
            // optional L2 prefetch cursor: runs `pair_prefetch` contraction blocks ahead of the load cursor (across tile boundaries)
            int pf_tile = first_tile, pf_kb = 0, pf_m0 = 0, pf_n0 = 0;
            auto pf_origin = [&]() {
                const PairTile t = pair_tile(p, pf_tile);
                pf_m0 = t.m0 + static_cast<int>(rank) * 128;
                pf_n0 = t.n0 + static_cast<int>(rank) * 128;
            };
            auto pf_step = [&]() {
                if (pf_tile >= num_tiles) return;
                const int k0 = pf_kb * BK;
                if (!p.a_mn) tma_prefetch_l2_2d(&tmA, k0, pf_m0);
                else for (int c = 0; c < a_chunks; ++c) tma_prefetch_l2_2d(&tmA, pf_m0 + c * BK, k0);
                if (!p.b_mn) tma_prefetch_l2_2d(&tmB, k0, pf_n0);
                else for (int c = 0; c < b_chunks; ++c) tma_prefetch_l2_2d(&tmB, pf_n0 + c * BK, k0);
                if (++pf_kb == num_k) {
                    pf_kb = 0;
                    pf_tile += tile_step;
                    if (pf_tile < num_tiles) pf_origin();
                }
            };
            if (p.pair_prefetch > 0 && first_tile < num_tiles) {
                pf_origin();
                for (int i = 0; i < PAIR_STAGES + p.pair_prefetch; ++i) pf_step();
            }
            for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
                const PairTile t = pair_tile(p, tile);
                const int m0 = t.m0 + static_cast<int>(rank) * 128, n0 = t.n0 + static_cast<int>(rank) * 128;
                for (int kb = 0; kb < num_k; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, &abort_flag)) { ok = false; break; }
                    if (p.pair_prefetch > 0) pf_step();
                    const uint32_t sa = smem_base + stage * PAIR_STAGE_BYTES;
                    const uint32_t sb = sa + A_STAGE_BYTES;
                    const uint32_t bar = mapa_shared(full_bar(stage), 0);                 // the leader's barrier counts both CTAs' bytes
                    if (leader) mbar_expect_tx(full_bar(stage), 2 * PAIR_STAGE_BYTES);
                    const int k0 = kb * BK;
                    if (!p.a_mn) {
                        tma_load_2d_pair(sa, &tmA, k0, m0, bar);
                    } else {
                        for (int c = 0; c < a_chunks; ++c) tma_load_2d_pair(sa + c * chunk_bytes, &tmA, m0 + c * BK, k0, bar);
                    }
                    if (!p.b_mn) {
                        tma_load_2d_pair(sb, &tmB, k0, n0, bar);
                    } else {
                        for (int c = 0; c < b_chunks; ++c) tma_load_2d_pair(sb + c * chunk_bytes, &tmB, n0 + c * BK, k0, bar);
                    }
                    if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (leader && elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t acc_phase[2] = {0, 0};
            int local_tile = 0;
            const uint32_t idesc = make_idesc(p.a_fmt, p.b_fmt, p.a_mn, p.b_mn, PAIR_BM, PAIR_BN);
            const uint32_t lbo = BK * TILE_K_BYTES;
            const uint32_t a_kstep = p.a_mn ? (BK / 4) * TILE_K_BYTES : 32;
            const uint32_t b_kstep = p.b_mn ? (BK / 4) * TILE_K_BYTES : 32;
            bool ok = true;
            for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++local_tile) {
                const int acc = local_tile & 1;
                if (!mbar_wait_cluster(tempty_bar(acc), acc_phase[acc] ^ 1u, &abort_flag)) { ok = false; break; }
                acc_phase[acc] ^= 1u;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * PAIR_BN;
                for (int kb = 0; kb < num_k; ++kb) {
                    if (!mbar_wait_cluster(full_bar(stage), phase, &abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_base + stage * PAIR_STAGE_BYTES;
                    const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t da = make_smem_desc(sa + j * a_kstep, p.a_mn ? lbo : 16, 1024);
                        const uint64_t db = make_smem_desc(sb + j * b_kstep, p.b_mn ? lbo : 16, 1024);
                        const uint32_t accum = (kb > 0 || j > 0) ? 1u : 0u;
                        if (p.elem_bytes == 2) mma_f16_pair(d_tmem, da, db, idesc, accum);
                        else mma_f8_pair(d_tmem, da, db, idesc, accum);
                    }
                    tc_commit_pair(empty_bar(stage), 3);   // both CTAs' stage is free once these MMAs have read it
                    if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) tc_commit_pair(tfull_bar(acc), 3);  // both CTAs' halves of the accumulator are complete
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs; each CTA drains its own 128 rows)
        const int quad = warp & 3;
        uint32_t acc_phase[2] = {0, 0};
        int local_tile = 0;
        float scale = p.alpha;
        if (p.scale_a) scale *= __ldg(p.scale_a);
        if (p.scale_b) scale *= __ldg(p.scale_b);
        float amax = 0.f;
        bool ok = true;
        const uint32_t tempty_leader[2] = {mapa_shared(tempty_bar(0), 0), mapa_shared(tempty_bar(1), 0)};
        const uint32_t stage_smem = epi_base + quad * PAIR_EPI_WARP_BYTES;
        uint8_t* stage_ptr = smem_raw + (stage_smem - smem_u32(smem_raw));
        int buf = 0, stores_in_flight = 0;
        for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++local_tile) {
            const PairTile pt = pair_tile(p, tile);
            const int acc = local_tile & 1;
            if (!mbar_wait(tfull_bar(acc), acc_phase[acc], &abort_flag)) { ok = false; break; }
            acc_phase[acc] ^= 1u;
            tc_fence_after();
            const int row_w = pt.m0 + static_cast<int>(rank) * 128 + quad * 32;   // first row of this warp
            const uint32_t t_row = tmem_base + acc * PAIR_BN + (static_cast<uint32_t>(quad * 32) << 16);
            if (use_tma_store) {
                const int cols_per_store = p.out_fp32 ? 32 : 64;
                if (row_w < p.M) {
#pragma unroll 1
                    for (int c = 0; c < PAIR_BN && pt.n0 + c < p.N; c += cols_per_store) {
                        uint32_t r0[32], r1[32];
                        tmem_ld_32x32(t_row + c, r0);
                        if (!p.out_fp32) tmem_ld_32x32(t_row + c + 32, r1);
                        if (stores_in_flight >= 2) {      // the store that last read this staging tile has finished reading it
                            if (lane == 0) tma_store_wait_read<1>();
                            __syncwarp();
                        }
                        tmem_ld_wait();
                        uint8_t* srow = stage_ptr + buf * 4096 + lane * 128;
                        if (p.out_fp32) {
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const float4 v = make_float4(__uint_as_float(r0[u * 4]) * scale, __uint_as_float(r0[u * 4 + 1]) * scale,
                                                             __uint_as_float(r0[u * 4 + 2]) * scale, __uint_as_float(r0[u * 4 + 3]) * scale);
                                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                                *reinterpret_cast<float4*>(srow + ((u ^ (lane & 7)) << 4)) = v;
                            }
                        } else {
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                uint4 o;
                                __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const int e = (u & 3) * 8 + 2 * i;
                                    const float a = __uint_as_float(u < 4 ? r0[e] : r1[e]) * scale, b = __uint_as_float(u < 4 ? r0[e + 1] : r1[e + 1]) * scale;
                                    amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
                                    pb[i] = __floats2bfloat162_rn(a, b);
                                }
                                *reinterpret_cast<uint4*>(srow + ((u ^ (lane & 7)) << 4)) = o;
                            }
                        }
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            if (p.accumulate) tma_reduce_add_2d(&tmD, stage_smem + buf * 4096, pt.n0 + c, row_w);
                            else tma_store_2d(&tmD, stage_smem + buf * 4096, pt.n0 + c, row_w);
                            tma_store_commit();
                        }
                        ++stores_in_flight;
                        buf ^= 1;
                    }
                }
            } else {
                TileInfo t;
                t.m_end = p.M;
                t.n_end = p.N;
                t.d_off = 0;
                const int row = row_w + lane;
#pragma unroll 1
                for (int c = 0; c < PAIR_BN; c += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(t_row + c, r);
                    tmem_ld_wait();
                    store_direct_32(p, t, row, pt.n0 + c, r, scale, amax);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader[acc]);
        }
        if (use_tma_store && lane == 0) tma_store_wait_all();
        if (p.amax_out) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (lane == 0 && amax > 0.f) atomicMax(reinterpret_cast<unsigned int*>(p.amax_out), __float_as_uint(amax));
        }
    }

    tc_fence_before();
    cluster_sync_all();   // neither CTA leaves (or frees TMEM) while the other may still signal its barriers or read its shared memory
    if (threadIdx.x == 0 && abort_flag && p.error_flag) atomicExch(p.error_flag, 1);
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// ------------------------------------------------------------------------------------------------ host side
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn get_encode_fn() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !ptr)
            return nullptr;
        fn = reinterpret_cast<EncodeFn>(ptr);
    }
    return fn;
}

const char* make_tensor_map_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                               uint32_t box_inner, uint32_t box_outer) {
    EncodeFn enc = get_encode_fn();
    if (!enc) return "cuTensorMapEncodeTiled unavailable";
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return "TMA base address must be 16-byte aligned";
    if (row_stride_bytes % 16 != 0) return "TMA row stride must be a multiple of 16 bytes";
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
    CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? nullptr : "cuTensorMapEncodeTiled failed";
}

template <int BN> static const char* launch(const GemmOperand& A, const GemmOperand& B, const GemmParams& p, int num_sms, cudaStream_t stream) {
    using C = Cfg<BN>;
    const int BK = TILE_K_BYTES / p.elem_bytes;
    CUtensorMap tmA, tmB;
    const char* e;
    // K-major: inner = K, outer = rows, box {BK, rows_per_tile}.  MN-major: inner = rows, outer = K, box {128 B of rows, BK}.
    // Extents of the stored 2-D operands.  Grouped modes: a_rows / b_rows are the totals over all groups.
    const uint64_t a_rows = p.mode == 0 ? (p.a_mn ? p.K : p.M) : p.a_total_rows;
    const uint64_t b_rows = p.mode == 0 ? (p.b_mn ? p.K : p.N) : p.b_total_rows;
    if (!p.a_mn) e = make_tensor_map_2d(&tmA, A.ptr, p.elem_bytes, p.K, a_rows, A.row_stride_bytes, BK, BM);
    else e = make_tensor_map_2d(&tmA, A.ptr, p.elem_bytes, p.M, a_rows, A.row_stride_bytes, BK, BK);
    if (e) return e;
    if (!p.b_mn) e = make_tensor_map_2d(&tmB, B.ptr, p.elem_bytes, p.K, b_rows, B.row_stride_bytes, BK, BN);
    else e = make_tensor_map_2d(&tmB, B.ptr, p.elem_bytes, p.N, b_rows, B.row_stride_bytes, BK, BK);
    if (e) return e;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
            return "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed";
        attr_set = true;
    }
    const int num_tiles = p.mode == 0 ? ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) : num_sms;  // grouped: tile count lives on the device
    const int grid = num_tiles < num_sms ? num_tiles : num_sms;
    gemm_tcgen05_kernel<BN><<<grid, GEMM_THREADS, C::SMEM_BYTES, stream>>>(tmA, tmB, p);
    return cudaGetLastError() == cudaSuccess ? nullptr : "gemm kernel launch failed";
}

static const char* launch_pair(const GemmOperand& A, const GemmOperand& B, GemmParams p, int num_sms, cudaStream_t stream) {
    const int BK = TILE_K_BYTES / p.elem_bytes;
    // L2 prefetch is off unless asked for: measured on B200 it costs 3-5 % (the kernel is bound by operand delivery bandwidth, not by
    // DRAM latency: four, five and six ring stages run at the same speed, half the operand bytes run 15-18 % faster)
    if (p.pair_group_m <= 0) {
        // The group's A panel (group_m x 256 rows x K) is re-read from L2 by every tile of the sweep over N while B streams through
        // once per group: make the panel as tall as a quarter of the L2 allows, so B is fetched from DRAM as few times as possible.
        const long long panel_row_bytes = static_cast<long long>(PAIR_BM) * p.K * p.elem_bytes;
        long long g = (32ll << 20) / (panel_row_bytes > 0 ? panel_row_bytes : 1);
        g = g < 4 ? 4 : (g > 32 ? 32 : g);
        p.pair_group_m = static_cast<int>(g);
    }
    CUtensorMap tmA, tmB, tmD;
    const char* e;
    if (!p.a_mn) e = make_tensor_map_2d(&tmA, A.ptr, p.elem_bytes, p.K, p.M, A.row_stride_bytes, BK, BM);
    else e = make_tensor_map_2d(&tmA, A.ptr, p.elem_bytes, p.M, p.K, A.row_stride_bytes, BK, BK);
    if (e) return e;
    if (!p.b_mn) e = make_tensor_map_2d(&tmB, B.ptr, p.elem_bytes, p.K, p.N, B.row_stride_bytes, BK, 128);
    else e = make_tensor_map_2d(&tmB, B.ptr, p.elem_bytes, p.N, p.K, B.row_stride_bytes, BK, BK);
    if (e) return e;
    // The shared-memory epilogue serves plain stores and fp32 accumulation (TMA add).  bf16 accumulation (D is read, summed in
    // fp32 and rounded once) and an abs-max that must include the accumulated values stay on the register path.
    const int d_bytes = p.out_fp32 ? 4 : 2;
    int use_tma_store = (!p.accumulate || (p.out_fp32 && !p.amax_out)) && (static_cast<uint64_t>(p.ldd) * d_bytes) % 16 == 0;
    if (use_tma_store) {
        e = make_tensor_map_2d(&tmD, p.D, d_bytes, p.N, p.M, static_cast<uint64_t>(p.ldd) * d_bytes, 128 / d_bytes, 32);
        if (e) use_tma_store = 0;
    }
    if (!use_tma_store) tmD = tmA;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES) != cudaSuccess)
            return "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed (pair GEMM)";
        attr_set = true;
    }
    const int num_tiles = ((p.M + PAIR_BM - 1) / PAIR_BM) * ((p.N + PAIR_BN - 1) / PAIR_BN);
    const int clusters = num_tiles < num_sms / 2 ? num_tiles : num_sms / 2;
    gemm_pair_kernel<<<2 * clusters, GEMM_THREADS, PAIR_SMEM_BYTES, stream>>>(tmA, tmB, tmD, p, use_tma_store);
    return cudaGetLastError() == cudaSuccess ? nullptr : "pair gemm kernel launch failed";
}

const char* gemm_sm100(const GemmOperand& A, const GemmOperand& B, GemmParams p, int num_sms, cudaStream_t stream) {
    if (p.M <= 0 || p.N <= 0 || p.K <= 0) return nullptr;
    if (p.mode != 0 && (p.num_groups <= 0 || p.num_groups > MAX_GROUPS || !p.group_offsets)) return "gemm_sm100: grouped mode needs 1..256 groups and offsets";
    if (p.N % 8 != 0 || p.ldd % 8 != 0) return "gemm_sm100: N and ldd must be multiples of 8";
    if ((reinterpret_cast<uintptr_t>(p.D) & 15) != 0) return "gemm_sm100: D must be 16-byte aligned";
    // CTA pairs (256 x 256 per cluster) for dense problems with at least one tile per cluster; tile_n = 512 forces them, 128 / 256
    // force the single-CTA kernels
    const long tiles_pair = static_cast<long>((p.M + PAIR_BM - 1) / PAIR_BM) * ((p.N + PAIR_BN - 1) / PAIR_BN);
    if (p.mode == 0 && (p.tile_n == 512 || (p.tile_n == 0 && tiles_pair >= num_sms / 2))) return launch_pair(A, B, p, num_sms, stream);
    // 128-wide N tiles when the wide tile would leave SMs idle or N is small
    const long tiles256 = static_cast<long>((p.M + BM - 1) / BM) * ((p.N + 255) / 256);
    const bool narrow = p.N <= 128 || (p.tile_n == 128) || (p.tile_n == 0 && tiles256 < num_sms);
    return narrow ? launch<128>(A, B, p, num_sms, stream) : launch<256>(A, B, p, num_sms, stream);
}

}  // namespace sg

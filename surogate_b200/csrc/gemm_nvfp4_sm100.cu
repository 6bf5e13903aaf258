// NVFP4 block-scaled GEMM for sm_100a: D[M,N] (bf16) = alpha * sa * sb * sum_k (A_q * SFA)(B_q * SFB)^T.
//
// A [M, K] and B [N, K] hold packed E2M1 (two values per byte, K contiguous); SFA / SFB hold one UE4M3 scale per 16
// elements of K in the 128x4 atom layout (see nvfp4_kernels.cu).  The tensor core applies the block scales itself:
// tcgen05.mma kind::mxf4nvf4.block_scale reads the values from shared memory (TMA, 128-byte swizzle) and the scale
// factors from TMEM, where tcgen05.cp places them from shared memory just ahead of the MMAs that use them.
//
// Tiling: 128 x 128 output tile, 256 elements of K (128 bytes) per pipeline stage = 4 MMAs of K = 64; 5 stages;
// double-buffered accumulator (2 x 128 TMEM columns) + two 32-column scale-factor areas.  Same persistent,
// warp-specialised structure as the bf16 / FP8 kernel (TMA warp, MMA warp, 4 epilogue warps).
//
// Replaces the CUTLASS Sm100 block-scaled instantiation of the reference
// (csrc/src/recipes/nvfp4/kernels/matmul_cutlass_fp4_sm100.cu:41-159).
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace sg {

namespace fp4 {
constexpr int BM = 128, BN = 128;
constexpr int ROW_BYTES = 128;                    // 256 fp4 values of K per stage
constexpr int A_BYTES = BM * ROW_BYTES, B_BYTES = BN * ROW_BYTES;
constexpr int SF_BYTES = 4 * 512;                 // 4 atoms (128 rows x 4 blocks each) per stage and operand
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + 2 * SF_BYTES;
constexpr int STAGES = 5;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;                    // 2 x 128 accumulator + 2 x 32 scale factors, rounded to a power of two
constexpr int SF_TMEM_BASE = 256;
constexpr int GROUP_M = 8;
}  // namespace fp4

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, replicated into the four 32-lane quadrants
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t saddr) {
    // no swizzle; rows of 16 bytes, 8-row groups 128 bytes apart
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(16u >> 4) << 16;
    d |= static_cast<uint64_t>(128u >> 4) << 32;
    d |= 1ull << 46;
    return d;
}
__device__ __forceinline__ void mma_nvfp4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
}
// E2M1 x E2M1, UE4M3 scales, fp32 accumulate, K-major operands
__host__ __device__ constexpr uint32_t make_idesc_nvfp4(uint32_t M, uint32_t N) {
    return (1u << 7) | (1u << 10) | ((N >> 3) << 17) | (0u << 23) | ((M >> 4) << 24);
}

struct Fp4Params {
    int M, N, K;            // K in elements (multiple of 256)
    const uint8_t* sfa;     // atom layout, rows padded to 128, K blocks padded to 4
    const uint8_t* sfb;
    void* D;
    int ldd;
    int accumulate;
    int out_fp32;
    float alpha;
    const float* scale_a;
    const float* scale_b;
    int* error_flag;
};

__global__ void __launch_bounds__(fp4::THREADS, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Fp4Params p) {
    using namespace fp4;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_k = p.K / 256;
    const int atoms_k = (p.K / 16 + 3) / 4;
    const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
    const int num_tiles = num_m * num_n;
    auto tile_of = [&](int tile, int& m_blk, int& n_blk) {
        const int per_group = GROUP_M * num_n;
        const int group = tile / per_group;
        const int first_m = group * GROUP_M;
        const int gsize = min(num_m - first_m, GROUP_M);
        const int r = tile - group * per_group;
        m_blk = first_m + r % gsize;
        n_blk = r / gsize;
    };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 128); }
        fence_barrier_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 2) { tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int m_blk, n_blk;
                tile_of(tile, m_blk, n_blk);
                for (int kb = 0; kb < num_k; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, &abort_flag)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * STAGE_BYTES, sb = sa + A_BYTES, ssa = sb + B_BYTES, ssb = ssa + SF_BYTES;
                    mbar_expect_tx(full_bar(stage), STAGE_BYTES);
                    tma_load_2d(sa, &tmA, kb * ROW_BYTES, m_blk * BM, full_bar(stage));
                    tma_load_2d(sb, &tmB, kb * ROW_BYTES, n_blk * BN, full_bar(stage));
                    bulk_load_1d(ssa, p.sfa + (static_cast<size_t>(m_blk) * atoms_k + kb * 4) * 512, SF_BYTES, full_bar(stage));
                    bulk_load_1d(ssb, p.sfb + (static_cast<size_t>(n_blk) * atoms_k + kb * 4) * 512, SF_BYTES, full_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t acc_phase[2] = {0, 0};
            int local_tile = 0, sf_slot = 0;
            const uint32_t idesc = make_idesc_nvfp4(BM, BN);
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
                const int acc = local_tile & 1;
                if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, &abort_flag)) { ok = false; break; }
                acc_phase[acc] ^= 1u;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_k; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, &abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_base + stage * STAGE_BYTES, sb = sa + A_BYTES, ssa = sb + B_BYTES, ssb = ssa + SF_BYTES;
                    const uint32_t t_sfa = tmem_base + SF_TMEM_BASE + sf_slot * 32, t_sfb = t_sfa + 16;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {   // scale factors of the stage's four K = 64 steps
                        tmem_cp_32x128b_warpx4(t_sfa + 4 * j, make_sf_desc(ssa + 512 * j));
                        tmem_cp_32x128b_warpx4(t_sfb + 4 * j, make_sf_desc(ssb + 512 * j));
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t da = make_smem_desc(sa + j * 32, 16, 1024);
                        const uint64_t db = make_smem_desc(sb + j * 32, 16, 1024);
                        mma_nvfp4(d_tmem, da, db, idesc, t_sfa + 4 * j, t_sfb + 4 * j, (kb > 0 || j > 0) ? 1u : 0u);
                    }
                    tc_commit(empty_bar(stage));
                    sf_slot ^= 1;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) tc_commit(tfull_bar(acc));
            }
        }
    } else {
        const int quad = warp & 3;
        uint32_t acc_phase[2] = {0, 0};
        int local_tile = 0;
        float scale = p.alpha;
        if (p.scale_a) scale *= __ldg(p.scale_a);
        if (p.scale_b) scale *= __ldg(p.scale_b);
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
            int m_blk, n_blk;
            tile_of(tile, m_blk, n_blk);
            const int acc = local_tile & 1;
            if (!mbar_wait(tfull_bar(acc), acc_phase[acc], &abort_flag)) { ok = false; break; }
            acc_phase[acc] ^= 1u;
            tc_fence_after();
            const int row = m_blk * BM + quad * 32 + lane;
            const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld_32x32(t_row + c, r);
                tmem_ld_wait();
                const int col0 = n_blk * BN + c;
                if (row < p.M && col0 < p.N) {
                    if (p.out_fp32) {
                        float* drow = reinterpret_cast<float*>(p.D) + static_cast<size_t>(row) * p.ldd + col0;
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            if (col0 + g * 4 < p.N) {
                                float4 v = make_float4(__uint_as_float(r[g * 4]) * scale, __uint_as_float(r[g * 4 + 1]) * scale,
                                                       __uint_as_float(r[g * 4 + 2]) * scale, __uint_as_float(r[g * 4 + 3]) * scale);
                                float4* dst = reinterpret_cast<float4*>(drow + g * 4);
                                if (p.accumulate) { const float4 o = *dst; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
                                *dst = v;
                            }
                        }
                    } else {
                        __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<size_t>(row) * p.ldd + col0;
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            if (col0 + g * 8 < p.N) {
                                float v[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]) * scale;
                                uint4* dst = reinterpret_cast<uint4*>(drow + g * 8);
                                if (p.accumulate) {
                                    const uint4 o = *dst;
                                    const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
                                    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(ob[i]); v[2 * i] += f.x; v[2 * i + 1] += f.y; }
                                }
                                uint4 out;
                                __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                                for (int i = 0; i < 4; ++i) pb[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                                *dst = out;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(tempty_bar(acc));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag && p.error_flag) atomicExch(p.error_flag, 1);
    if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, fp4::TMEM_COLS); }
}

const char* gemm_nvfp4_sm100(const void* a, const void* b, const void* sfa, const void* sfb, void* d, int M, int N, int K, int ldd, int out_fp32,
                             int accumulate, float alpha, const float* scale_a, const float* scale_b, int* error_flag, int num_sms,
                             cudaStream_t stream) {
    using namespace fp4;
    if (M <= 0 || N <= 0 || K <= 0) return nullptr;
    if (K % 256 != 0) return "gemm_nvfp4: K must be a multiple of 256";
    if (N % 8 != 0 || ldd % 8 != 0) return "gemm_nvfp4: N and ldd must be multiples of 8";
    CUtensorMap tmA, tmB;
    const char* e = make_tensor_map_2d(&tmA, a, 1, static_cast<uint64_t>(K) / 2, M, static_cast<uint64_t>(K) / 2, ROW_BYTES, BM);
    if (e) return e;
    e = make_tensor_map_2d(&tmB, b, 1, static_cast<uint64_t>(K) / 2, N, static_cast<uint64_t>(K) / 2, ROW_BYTES, BN);
    if (e) return e;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_nvfp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
            return "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed";
        attr_set = true;
    }
    Fp4Params p{};
    p.M = M; p.N = N; p.K = K;
    p.sfa = static_cast<const uint8_t*>(sfa);
    p.sfb = static_cast<const uint8_t*>(sfb);
    p.D = d; p.ldd = ldd; p.accumulate = accumulate; p.out_fp32 = out_fp32; p.alpha = alpha;
    p.scale_a = scale_a; p.scale_b = scale_b; p.error_flag = error_flag;
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    gemm_nvfp4_kernel<<<tiles < num_sms ? tiles : num_sms, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
    return cudaGetLastError() == cudaSuccess ? nullptr : "gemm_nvfp4 kernel launch failed";
}

}  // namespace sg

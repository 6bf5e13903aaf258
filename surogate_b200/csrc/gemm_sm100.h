// Host API of the sm_100a tcgen05 GEMM (see gemm_sm100.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sg {

struct GemmOperand {
    const void* ptr;            // first element of the 2-D view
    uint64_t row_stride_bytes;  // stride between rows of the stored matrix (inner dimension is contiguous)
};

struct GemmParams {
    int M, N, K;
    int elem_bytes;   // 2 = bf16 (kind::f16), 1 = fp8 (kind::f8f6f4)
    int a_fmt, b_fmt; // bf16: 1 ; fp8: 0 = e4m3, 1 = e5m2
    int a_mn, b_mn;   // 0: operand stored [rows, K] (K-major); 1: stored [K, rows] (MN-major)
    void* D;          // [M, N] row-major, leading dimension ldd (elements)
    int ldd;
    int out_fp32;     // 0: bf16 output, 1: fp32 output
    int accumulate;   // 1: D += result
    float alpha;
    const float* scale_a;  // optional device scalars multiplied into the result (FP8 de-scales)
    const float* scale_b;
    float* amax_out;       // optional: running max |D| (atomicMax on the bit pattern)
    int* error_flag;       // set to 1 if a pipeline wait ran out of budget
    int tile_n;            // 0 = auto; 128 / 256 = single-CTA tiles of that width; 512 = 256 x 256 tiles on CTA pairs
    int pair_prefetch;     // CTA-pair kernel: L2 prefetch distance in contraction blocks beyond the shared-memory ring (<= 0 = off, the default)
    int pair_group_m;      // CTA-pair kernel: 256-row tiles per rasterisation group (0 = chosen from the operand sizes)
    // Grouped problems (MoE).  mode 0: dense.  mode 1: rows of A and D are grouped, group g = rows [offs[g], offs[g+1]) (each a
    // multiple of 128) and multiplies weight block g (M is unused; N, K are per-group sizes).  mode 2: the contraction is grouped:
    // output matrix g [M, N] = A[rows of g]^T . B[rows of g] (both operands MN-major, stored [total_rows, M] / [total_rows, N]).
    int mode;
    int num_groups;
    const int* group_offsets;    // device, num_groups + 1 entries
    long long a_total_rows;      // stored rows of A (grouped modes)
    long long b_total_rows;      // stored rows of B (grouped modes)
};

const char* gemm_sm100(const GemmOperand& A, const GemmOperand& B, GemmParams p, int num_sms, cudaStream_t stream);

const char* make_tensor_map_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                               uint32_t box_inner, uint32_t box_outer);

}  // namespace sg

namespace sg {
// NVFP4 block-scaled GEMM (gemm_nvfp4_sm100.cu): a [M, K/2] and b [N, K/2] packed E2M1, sfa / sfb UE4M3 scales in atom layout.
const char* gemm_nvfp4_sm100(const void* a, const void* b, const void* sfa, const void* sfb, void* d, int M, int N, int K, int ldd, int out_fp32,
                             int accumulate, float alpha, const float* scale_a, const float* scale_b, int* error_flag, int num_sms,
                             cudaStream_t stream);
}  // namespace sg

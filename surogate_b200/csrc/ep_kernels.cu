// Expert-parallel dispatch / combine over peer-mapped memory (NVLink through NVSwitch), fused with the routing
// permutation and the weighted combine:
//
//   ep_plan     : every rank publishes its per-expert token counts into all peers' tables (P2P stores), a flag
//                 barrier follows inside the kernel, then each rank derives (a) the padded row layout of its own
//                 experts' receive buffer and (b) the first row it may write for every (global) expert on its owner.
//   ep_dispatch : one CTA per token; each of the token's K copies takes its precomputed row on the expert's owner and the
//                 token's activation row is stored straight into the owner's receive buffer (16-byte P2P stores),
//                 optionally scaled (backward: d_yp = w * dy).  This is routing permutation + all-to-all in one pass.
//   ep_combine  : one CTA per token; pulls its K expert-output rows from the owners (P2P loads) and forms the
//                 weighted sum; optionally keeps the pulled rows (they are what backward needs for d_weights).
//
// All waits on peers are bounded and report through the error word.  No TMA touches peer memory.
//
// Replaces csrc/src/runtime/ep/ep_strategy.cpp:621-856 (split exchange + grouped ncclSend/Recv + host syncs) and
// csrc/src/kernels/ep_dispatch.cu of the reference.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_kernels.h"
#include "ep_kernels.h"

namespace sg {

using bf16 = __nv_bfloat16;
using bf162 = __nv_bfloat162;

__device__ __forceinline__ void ep_st_release(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ep_ld_acquire(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// ctrl layout per rank (ints): [0, W*E) all_counts[src][expert] ; pads (uint32) live in the communicator's signal pad.
// Outputs (local, ints): offsets[2*El+2] = padded start rows of my experts (El+1 entries, clamped to the buffer), overflow rows,
// then the real row count of each of my experts; dst_base[E] (first row I may write per global expert),
// cursors[E] = 0.
__global__ void __launch_bounds__(256) ep_plan_kernel(PeerPtrs ctrl, PeerPtrs pads, const int* __restrict__ counts, int* __restrict__ offsets,
                                                      int* __restrict__ dst_base, int* __restrict__ cursors, int E, int rank, int world,
                                                      uint32_t epoch, int slot_base, int capacity_rows, int* error_flag, long long budget) {
    const int El = E / world;
    const int t = threadIdx.x;
    // 1. publish my counts to every rank's table
    for (int i = t; i < E * world; i += blockDim.x) {
        const int dst = i / E, e = i - dst * E;
        reinterpret_cast<int*>(ctrl.p[dst])[rank * E + e] = counts[e];
    }
    __threadfence_system();
    __syncthreads();
    __shared__ int failed;
    if (t == 0) failed = 0;
    __syncthreads();
    if (t < world) {
        ep_st_release(reinterpret_cast<uint32_t*>(pads.p[t]) + slot_base + rank, epoch);
        const uint32_t* w = reinterpret_cast<const uint32_t*>(pads.p[rank]) + slot_base + t;
        const long long t0 = clock64();
        while (static_cast<int32_t>(ep_ld_acquire(w) - epoch) < 0) {
            if (clock64() - t0 > budget) { atomicExch(error_flag, 2); failed = 1; break; }
            __nanosleep(32);
        }
    }
    __syncthreads();
    if (failed) return;
    // 2. every rank now holds all_counts[src][e] for all sources and experts
    const volatile int* all = reinterpret_cast<const volatile int*>(ctrl.p[rank]);
    __shared__ int tot[256];     // total rows per global expert
    for (int e = t; e < E; e += blockDim.x) {
        int s = 0;
        for (int r = 0; r < world; ++r) s += all[r * E + e];
        tot[e] = s;
        cursors[e] = 0;
    }
    __syncthreads();
    for (int e = t; e < E; e += blockDim.x) {
        const int owner = e / El, el = e - owner * El;
        int off = 0;
        for (int j = 0; j < el; ++j) off += (tot[owner * El + j] + 127) / 128 * 128;   // padded start of this expert on its owner
        int before = 0;
        for (int r = 0; r < rank; ++r) before += all[r * E + e];                       // rows of lower-ranked sources come first
        dst_base[e] = off + before;   // rows at or beyond capacity_rows are dropped by the dispatch kernel (token dropping)
        // The grouped GEMMs walk offsets[]: clamp them so that nothing beyond the receive buffer is ever touched.
        if (owner == rank) offsets[el] = off < capacity_rows ? off : capacity_rows;
        if (owner == rank && el == El - 1) {
            const int end = off + (tot[e] + 127) / 128 * 128;
            offsets[El] = end < capacity_rows ? end : capacity_rows;
            offsets[El + 1] = end > capacity_rows ? end - capacity_rows : 0;           // rows that did not fit (statistics)
        }
        if (owner == rank) offsets[El + 2 + el] = tot[e];                              // real (unpadded) rows of my expert el
    }
}

// Zero the padding rows of every local expert's region (rows [start + real, next start), inside the buffer).  Only padding is
// touched, so it is safe while peers are already storing real rows.
__global__ void __launch_bounds__(256) ep_zero_pad_rows_kernel(bf16* __restrict__ buf, const int* __restrict__ offsets, int El, int C, int capacity_rows) {
    const int el = blockIdx.y;
    const int lo = min(offsets[el] + offsets[El + 2 + el], capacity_rows), hi = min(offsets[el + 1], capacity_rows);
    const int vec_per_row = C / 8;
    const long long total = static_cast<long long>(hi - lo) * vec_per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x)
        reinterpret_cast<uint4*>(buf + static_cast<size_t>(lo) * C)[i] = make_uint4(0, 0, 0, 0);
}

// dst[0:n) = src[0:n) rows, n read from device memory (the padded row count of this step): cost follows the rows in use, not
// the capacity of the buffer.
__global__ void __launch_bounds__(256) copy_rows_upto_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const int* __restrict__ n_rows, int C) {
    const long long total = static_cast<long long>(*n_rows) * (C / 8);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) dst[i] = src[i];
}

// Position of every (token, k) copy among this rank's copies for the same expert, in token order: a stable counting sort done by
// one CTA per expert (ballot + running count).  Replaces claiming rows with atomics, so the row order inside an expert, and with
// it the summation order of the weight gradients, is the same in every run.
__global__ void __launch_bounds__(256) ep_row_positions_kernel(const int* __restrict__ topk_idx, int* __restrict__ pos, int n_entries) {
    __shared__ int warp_count[8];
    __shared__ int running;
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) running = 0;
    __syncthreads();
    for (int base = 0; base < n_entries; base += 256) {
        const int i = base + threadIdx.x;
        const bool mine = i < n_entries && topk_idx[i] == e;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_count[warp] = __popc(m);
        __syncthreads();
        int before = running;
        for (int w = 0; w < warp; ++w) before += warp_count[w];
        if (mine) pos[i] = before + __popc(m & ((1u << lane) - 1u));
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
            for (int w = 0; w < 8; ++w) t += warp_count[w];
            running += t;
        }
        __syncthreads();
    }
}

// x [tokens, C] bf16; recv = peers' receive buffers ([capacity, C] each).  row_map[tok*K+k] = owner * capacity + row (or -1).
// row_pos[tok*K+k] = position of the copy among this rank's copies for that expert (ep_row_positions_kernel).
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const bf16* __restrict__ x, const int* __restrict__ topk_idx, const float* __restrict__ w,
                                                          const int* __restrict__ dst_base, const int* __restrict__ row_pos, int* __restrict__ row_map,
                                                          PeerPtrs recv, int C, int K, int El, int capacity_rows, int reuse_map,
                                                          const float* __restrict__ q_scale, float* __restrict__ amax_out) {
    // q_scale != null: rows cross NVLink as E4M3 (value * *q_scale), one byte per element into a [capacity, C] byte buffer, and the
    // abs-max of what was sent is recorded for the next step's scale (delayed scaling; the scale is the same on every rank).
    __shared__ long long dst[16];
    __shared__ float ws[16];
    __shared__ float red[8];
    const int tok = blockIdx.x;
    if (threadIdx.x < K) {
        long long code = -1;
        if (reuse_map) {
            code = row_map[tok * K + threadIdx.x];
        } else {
            const int e = topk_idx[tok * K + threadIdx.x];
            const int row = dst_base[e] + row_pos[tok * K + threadIdx.x];
            if (row < capacity_rows) code = static_cast<long long>(e / El) * capacity_rows + row;
            row_map[tok * K + threadIdx.x] = static_cast<int>(code);
        }
        dst[threadIdx.x] = code;
        ws[threadIdx.x] = w ? w[tok * K + threadIdx.x] : 1.f;
    }
    __syncthreads();
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(tok) * C);
    if (q_scale) {
        const float qs = __ldg(q_scale);
        float amax = 0.f;
        for (int c = threadIdx.x; c < C / 8; c += blockDim.x) {
            const uint4 v = src[c];
            const bf162* p = reinterpret_cast<const bf162*>(&v);
            uint2 q;
            uint8_t* qb = reinterpret_cast<uint8_t*>(&q);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(p[i]);
                amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
                qb[2 * i] = __nv_cvt_float_to_fp8(f.x * qs, __NV_SATFINITE, __NV_E4M3);
                qb[2 * i + 1] = __nv_cvt_float_to_fp8(f.y * qs, __NV_SATFINITE, __NV_E4M3);
            }
            for (int k = 0; k < K; ++k) {
                if (dst[k] < 0) continue;
                const int owner = static_cast<int>(dst[k] / capacity_rows);
                const size_t row = static_cast<size_t>(dst[k] - static_cast<long long>(owner) * capacity_rows);
                reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(recv.p[owner]) + row * C)[c] = q;
            }
        }
        if (amax_out) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
                if (amax > 0.f) atomicMax(reinterpret_cast<unsigned int*>(amax_out), __float_as_uint(amax));
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < C / 8; c += blockDim.x) {
        const uint4 v = src[c];
        for (int k = 0; k < K; ++k) {
            if (dst[k] < 0) continue;
            const int owner = static_cast<int>(dst[k] / capacity_rows);
            const size_t row = static_cast<size_t>(dst[k] - static_cast<long long>(owner) * capacity_rows);
            uint4 o = v;
            if (w) {
                const bf162* p = reinterpret_cast<const bf162*>(&v);
                bf162* po = reinterpret_cast<bf162*>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(p[i]);
                    po[i] = __floats2bfloat162_rn(f.x * ws[k], f.y * ws[k]);
                }
            }
            reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(recv.p[owner]) + row * C)[c] = o;
        }
    }
}

// y[tok] = sum_k w[tok,k] * out_owner[row] ; optionally rows_out[tok*K+k] = out_owner[row].  All of a token's peer loads (up to
// eight per trip) are issued before the first is used, so their NVLink latencies overlap instead of adding up.
__global__ void __launch_bounds__(256) ep_combine_kernel(PeerPtrs outs, const float* __restrict__ w, const int* __restrict__ row_map,
                                                         bf16* __restrict__ y, bf16* __restrict__ rows_out, int C, int K, int capacity_rows) {
    __shared__ const bf16* src_row[16];
    __shared__ float ws[16];
    const int tok = blockIdx.x;
    if (threadIdx.x < K) {
        const int code = row_map[tok * K + threadIdx.x];
        const bf16* r = nullptr;
        if (code >= 0) {
            const int owner = code / capacity_rows;
            r = reinterpret_cast<const bf16*>(outs.p[owner]) + static_cast<size_t>(code - owner * capacity_rows) * C;
        }
        src_row[threadIdx.x] = r;
        ws[threadIdx.x] = w ? w[tok * K + threadIdx.x] : 1.f;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C / 8; c += blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k0 = 0; k0 < K; k0 += 8) {
            uint4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = make_uint4(0, 0, 0, 0);
                if (k0 + j < K && src_row[k0 + j] != nullptr) {
                    const void* src = src_row[k0 + j] + static_cast<size_t>(c) * 8;
                    asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v[j].x), "=r"(v[j].y), "=r"(v[j].z), "=r"(v[j].w) : "l"(src) : "memory");
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (k0 + j >= K) break;
                if (rows_out) reinterpret_cast<uint4*>(rows_out + (static_cast<size_t>(tok) * K + k0 + j) * C)[c] = v[j];
                const bf162* p = reinterpret_cast<const bf162*>(&v[j]);
                const float wk = ws[k0 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(p[i]);
                    acc[2 * i] += wk * f.x;
                    acc[2 * i + 1] += wk * f.y;
                }
            }
        }
        uint4 o;
        bf162* po = reinterpret_cast<bf162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        reinterpret_cast<uint4*>(y + static_cast<size_t>(tok) * C)[c] = o;
    }
}

// d_w[tok,k] = <rows[tok,k,:], dy[tok,:]>   (rows were kept by the forward combine)
__global__ void __launch_bounds__(256) ep_weight_grad_kernel(const bf16* __restrict__ rows, const bf16* __restrict__ dy, float* __restrict__ d_w, int C, int K) {
    __shared__ float red[16][8];
    const int tok = blockIdx.x;
    float dots[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) dots[k] = 0.f;
    for (int c = threadIdx.x; c < C / 8; c += blockDim.x) {
        const uint4 gv = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(tok) * C)[c];
        const bf162* gp = reinterpret_cast<const bf162*>(&gv);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            if (k >= K) break;
            const uint4 v = reinterpret_cast<const uint4*>(rows + (static_cast<size_t>(tok) * K + k) * C)[c];
            const bf162* p = reinterpret_cast<const bf162*>(&v);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 a = __bfloat1622float2(p[i]), b = __bfloat1622float2(gp[i]);
                dots[k] += a.x * b.x + a.y * b.y;
            }
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        if (k >= K) break;
        float s = dots[k];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) red[k][warp] = s;
    }
    __syncthreads();
    if (threadIdx.x < K) {
        float s = 0.f;
        for (int i = 0; i < (blockDim.x >> 5); ++i) s += red[threadIdx.x][i];
        d_w[tok * K + threadIdx.x] = s;
    }
}

void ep_plan(const PeerPtrs& ctrl, const PeerPtrs& pads, const int* counts, int* offsets, int* dst_base, int* cursors, int E, int rank, int world,
             uint32_t epoch, int slot_base, int capacity_rows, int* error_flag, double budget_s, cudaStream_t s) {
    ep_plan_kernel<<<1, 256, 0, s>>>(ctrl, pads, counts, offsets, dst_base, cursors, E, rank, world, epoch, slot_base, capacity_rows, error_flag,
                                     static_cast<long long>(budget_s * 2.0e9));
}
void ep_zero_pad_rows(void* buf, const int* offsets, int El, int C, int capacity_rows, cudaStream_t s) {
    ep_zero_pad_rows_kernel<<<dim3(8, El), 256, 0, s>>>((bf16*)buf, offsets, El, C, capacity_rows);
}
void copy_rows_upto(const void* src, void* dst, const int* n_rows, int C, int num_sms, cudaStream_t s) {
    copy_rows_upto_kernel<<<num_sms * 8, 256, 0, s>>>((const uint4*)src, (uint4*)dst, n_rows, C);
}
void ep_dispatch(const void* x, const int* topk_idx, const float* w, const int* dst_base, const int* row_pos, int* row_map, const PeerPtrs& recv, int tokens,
                 int C, int K, int El, int capacity_rows, int reuse_map, const float* q_scale, float* amax_out, cudaStream_t s) {
    ep_dispatch_kernel<<<tokens, 256, 0, s>>>((const bf16*)x, topk_idx, w, dst_base, row_pos, row_map, recv, C, K, El, capacity_rows, reuse_map, q_scale,
                                              amax_out);
}
void ep_row_positions(const int* topk_idx, int* pos, int n_entries, int E, cudaStream_t s) {
    ep_row_positions_kernel<<<E, 256, 0, s>>>(topk_idx, pos, n_entries);
}
void ep_combine(const PeerPtrs& outs, const float* w, const int* row_map, void* y, void* rows_out, int tokens, int C, int K, int capacity_rows,
                cudaStream_t s) {
    ep_combine_kernel<<<tokens, 256, 0, s>>>(outs, w, row_map, (bf16*)y, (bf16*)rows_out, C, K, capacity_rows);
}
void ep_weight_grad(const void* rows, const void* dy, float* d_w, int tokens, int C, int K, cudaStream_t s) {
    ep_weight_grad_kernel<<<tokens, 256, 0, s>>>((const bf16*)rows, (const bf16*)dy, d_w, C, K);
}

}  // namespace sg

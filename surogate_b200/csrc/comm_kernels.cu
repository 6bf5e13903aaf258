// Collective kernels over peer-mapped (symmetric) memory on an NVSwitch node.  Each GPU runs ONE kernel per
// collective; the kernel itself issues the loads from the peers' buffers (plain ld.global on peer-mapped
// addresses, or multimem.ld_reduce through the switch), so the data movement is fused with whatever is done
// to the data on arrival:
//
//   * reduce_scatter_fused: sum this rank's slice over all ranks' gradient buckets, scale, write the reduced
//     shard (bf16 or fp32) and accumulate the shard's sum of squares for the global gradient norm.
//   * all_gather_fused: pull every rank's weight shard and write it locally as bf16 and/or as FP8 with a
//     per-tensor scale (quantise-on-gather); the local FP8 copy is what the tcgen05 GEMMs read through TMA.
//   * all_reduce_small: latency-bound one-shot all-reduce for scalars / small vectors.
//   * barrier: flag exchange through each rank's signal pad.
//
// Cross-GPU waits are bounded: a rank that does not see its peers within the budget sets an error word that
// the host checks, and returns.  No TMA and no cluster multicast is used on peer memory anywhere.
//
// Replaces the NCCL call sites C1-C5 of the reference (csrc/src/utilities/comm.cpp:806-867) on the hot path.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_kernels.h"

namespace sg {

using bf16 = __nv_bfloat16;
using bf162 = __nv_bfloat162;

constexpr long long kPeerWaitCycles = 40000000000LL;  // ~20 s at 2 GHz: ranks may be skewed by a whole step

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_peer_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// ---------------------------------------------------------------------------------------- barrier
// pads[r] = rank r's signal pad (uint32 per peer).  Thread t tells rank t "I reached epoch e", then waits for rank t's word.
__global__ void symm_barrier_kernel(PeerPtrs pads, int rank, int world, uint32_t epoch, int slot_base, int* error_flag, long long budget) {
    const int t = threadIdx.x;
    if (t >= world) return;
    uint32_t* remote = reinterpret_cast<uint32_t*>(pads.p[t]) + slot_base + rank;
    __threadfence_system();
    st_release_sys(remote, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(pads.p[rank]) + slot_base + t;
    const long long t0 = clock64();
    // epochs only grow; signed distance handles wrap-around
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
        if (clock64() - t0 > budget) {
            atomicExch(error_flag, 2);
            return;
        }
        __nanosleep(64);
    }
}

// ---------------------------------------------------------------------------------------- reduce-scatter (+scale, +sumsq)
__device__ __forceinline__ void acc8(float (&a)[8], const uint4& v) {
    const bf162* p = reinterpret_cast<const bf162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(p[i]);
        a[2 * i] += f.x;
        a[2 * i + 1] += f.y;
    }
}

// bufs.p[r] + elem_offset = rank r's full gradient bucket (bf16).  This rank reduces elements [rank*S, (rank+1)*S).
template <bool OUT_FP32, bool ACCUMULATE, int U>
__global__ void __launch_bounds__(512) reduce_scatter_fused_kernel(PeerPtrs bufs, size_t elem_offset, size_t shard_elems, int rank, int world,
                                                                   float scale, void* __restrict__ out, float* __restrict__ sumsq_out) {
    // U output vectors per trip, world <= 8 / U: eight 16-byte peer loads are in flight per thread whatever the number of ranks
    // (NVLink round trips are microseconds; one load per thread leaves the links idle at 2 and 4 ranks)
    constexpr int R = 8 / U;
    __shared__ float sh[32];
    const size_t nvec = shard_elems / 8;
    const size_t base = elem_offset + static_cast<size_t>(rank) * shard_elems;
    const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
    float ss = 0.f;
    for (size_t v0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v0 < nvec; v0 += nthreads * U) {
        uint4 raw[U * R];
        // issue all peer loads first (independent, long latency over NVLink), then reduce in a fixed rank order
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t v = v0 + u * nthreads;
#pragma unroll
            for (int r = 0; r < R; ++r)
                if (r < world && v < nvec) raw[u * R + r] = ld_peer_16(reinterpret_cast<const bf16*>(bufs.p[r]) + base + v * 8);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t v = v0 + u * nthreads;
            if (v >= nvec) break;
            float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < R; ++r)
                if (r < world) acc8(a, raw[u * R + r]);
            if (OUT_FP32) {
                float* o = reinterpret_cast<float*>(out) + v * 8;
                float4 lo = make_float4(a[0] * scale, a[1] * scale, a[2] * scale, a[3] * scale);
                float4 hi = make_float4(a[4] * scale, a[5] * scale, a[6] * scale, a[7] * scale);
                if (ACCUMULATE) {
                    const float4 plo = *reinterpret_cast<const float4*>(o), phi = *reinterpret_cast<const float4*>(o + 4);
                    lo.x += plo.x; lo.y += plo.y; lo.z += plo.z; lo.w += plo.w;
                    hi.x += phi.x; hi.y += phi.y; hi.z += phi.z; hi.w += phi.w;
                }
                ss += lo.x * lo.x + lo.y * lo.y + lo.z * lo.z + lo.w * lo.w + hi.x * hi.x + hi.y * hi.y + hi.z * hi.z + hi.w * hi.w;
                *reinterpret_cast<float4*>(o) = lo;
                *reinterpret_cast<float4*>(o + 4) = hi;
            } else {
                uint4 o;
                bf162* po = reinterpret_cast<bf162*>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    po[i] = __floats2bfloat162_rn(a[2 * i] * scale, a[2 * i + 1] * scale);
                    const float2 f = __bfloat1622float2(po[i]);   // norm of what is actually stored
                    ss += f.x * f.x + f.y * f.y;
                }
                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(out) + v * 8) = o;
            }
        }
    }
    if (sumsq_out) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x < 32) {
            ss = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (threadIdx.x == 0) atomicAdd(sumsq_out, ss);
        }
    }
}

// NVLS variant: one multimem.ld_reduce per 16 bytes sums the same address on every GPU inside the switch.
template <bool OUT_FP32>
__global__ void __launch_bounds__(512) reduce_scatter_multimem_kernel(const void* mc_base, size_t elem_offset, size_t shard_elems, int rank, float scale,
                                                                      void* __restrict__ out, float* __restrict__ sumsq_out) {
    __shared__ float sh[32];
    const size_t nvec = shard_elems / 8;
    const bf16* src = reinterpret_cast<const bf16*>(mc_base) + elem_offset + static_cast<size_t>(rank) * shard_elems;
    float ss = 0.f;
    for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < nvec; v += static_cast<size_t>(gridDim.x) * blockDim.x) {
        uint4 r;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                     : "l"(src + v * 8)
                     : "memory");
        const bf162* p = reinterpret_cast<const bf162*>(&r);
        float a[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(p[i]);
            a[2 * i] = f.x * scale;
            a[2 * i + 1] = f.y * scale;
        }
        if (OUT_FP32) {
            float* o = reinterpret_cast<float*>(out) + v * 8;
            *reinterpret_cast<float4*>(o) = make_float4(a[0], a[1], a[2], a[3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(a[4], a[5], a[6], a[7]);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += a[i] * a[i];
        } else {
            uint4 o;
            bf162* po = reinterpret_cast<bf162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                po[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
                const float2 f = __bfloat1622float2(po[i]);
                ss += f.x * f.x + f.y * f.y;
            }
            *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(out) + v * 8) = o;
        }
    }
    if (sumsq_out) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x < 32) {
            ss = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (threadIdx.x == 0) atomicAdd(sumsq_out, ss);
        }
    }
}

// ---------------------------------------------------------------------------------------- all-gather (+quantise)
// Elements [seg_begin, seg_end) of the gathered bucket; element i lives on rank i / S at offset i % S of that rank's shard.
// Writes bf16 (out_bf16, bucket-relative) and/or FP8 e4m3 (out_fp8, bucket-relative) scaled by *scale.
__global__ void __launch_bounds__(512) all_gather_fused_kernel(PeerPtrs shards, size_t shard_elem_offset, size_t shard_elems, size_t seg_begin,
                                                               size_t seg_end, bf16* __restrict__ out_bf16, uint8_t* __restrict__ out_fp8,
                                                               const float* __restrict__ scale) {
    const float s = scale ? __ldg(scale) : 1.f;
    const size_t nvec = (seg_end - seg_begin) / 8;
    const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
    constexpr int U = 4;   // 16-byte peer loads in flight per thread: one load per thread leaves NVLink (microsecond round trips) idle
    for (size_t v0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v0 < nvec; v0 += nthreads * U) {
        uint4 raw[U];
        size_t idx[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t v = min(v0 + u * nthreads, nvec - 1);   // past the end: a duplicate of the last vector, not stored
            idx[u] = seg_begin + v * 8;
            const int r = static_cast<int>(idx[u] / shard_elems);
            const size_t local = idx[u] - static_cast<size_t>(r) * shard_elems;
            raw[u] = ld_peer_16(reinterpret_cast<const bf16*>(shards.p[r]) + shard_elem_offset + local);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (v0 + u * nthreads >= nvec) continue;
            const size_t i = idx[u];
            const uint4 rv = raw[u];
            if (out_bf16) *reinterpret_cast<uint4*>(out_bf16 + i) = rv;
            if (out_fp8) {
                const bf162* p = reinterpret_cast<const bf162*>(&rv);
                uint2 q;
                uint8_t* qb = reinterpret_cast<uint8_t*>(&q);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = __bfloat1622float2(p[k]);
                    qb[2 * k] = __nv_cvt_float_to_fp8(f.x * s, __NV_SATFINITE, __NV_E4M3);
                    qb[2 * k + 1] = __nv_cvt_float_to_fp8(f.y * s, __NV_SATFINITE, __NV_E4M3);
                }
                *reinterpret_cast<uint2*>(out_fp8 + i) = q;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------- small all-reduce (one shot)
// Each rank publishes its vector in its own symmetric slot, a flag exchange follows, then every rank reads all slots.
// n <= 1024 floats.  op: 0 = sum, 1 = max.
__global__ void __launch_bounds__(1024) all_reduce_small_kernel(PeerPtrs slots, PeerPtrs pads, size_t slot_elem_offset, float* __restrict__ data, int n,
                                                                int op, int rank, int world, uint32_t epoch, int slot_base, int* error_flag,
                                                                long long budget) {
    float* mine = reinterpret_cast<float*>(slots.p[rank]) + slot_elem_offset;
    for (int i = threadIdx.x; i < n; i += blockDim.x) mine[i] = data[i];
    __threadfence_system();
    __syncthreads();
    __shared__ int failed;
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    if (threadIdx.x < world) {
        const int t = threadIdx.x;
        st_release_sys(reinterpret_cast<uint32_t*>(pads.p[t]) + slot_base + rank, epoch);
        const uint32_t* w = reinterpret_cast<const uint32_t*>(pads.p[rank]) + slot_base + t;
        const long long t0 = clock64();
        while (static_cast<int32_t>(ld_acquire_sys(w) - epoch) < 0) {
            if (clock64() - t0 > budget) {
                atomicExch(error_flag, 2);
                failed = 1;
                break;
            }
            __nanosleep(32);
        }
    }
    __syncthreads();
    if (failed) return;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float acc = op == 1 ? -INFINITY : 0.f;
        for (int r = 0; r < world; ++r) {
            float v;
            const float* src = reinterpret_cast<const float*>(slots.p[r]) + slot_elem_offset + i;
            asm volatile("ld.global.relaxed.sys.f32 %0, [%1];" : "=f"(v) : "l"(src) : "memory");
            acc = op == 1 ? fmaxf(acc, v) : acc + v;
        }
        data[i] = acc;
    }
}

// ============================================================================================ launchers
static int comm_grid(size_t nvec, int threads, int max_blocks) {
    size_t g = (nvec + threads - 1) / threads;
    if (g < 1) g = 1;
    if (g > static_cast<size_t>(max_blocks)) g = max_blocks;
    return static_cast<int>(g);
}

void symm_barrier(const PeerPtrs& pads, int rank, int world, uint32_t epoch, int slot_base, int* error_flag, double budget_s, cudaStream_t s) {
    const long long budget = budget_s > 0 ? static_cast<long long>(budget_s * 2.0e9) : kPeerWaitCycles;
    symm_barrier_kernel<<<1, 32, 0, s>>>(pads, rank, world, epoch, slot_base, error_flag, budget);
}

void reduce_scatter_fused(const PeerPtrs& bufs, size_t elem_offset, size_t shard_elems, int rank, int world, float scale, void* out, int out_fp32,
                          int accumulate, float* sumsq_out, int max_blocks, cudaStream_t s) {
    const int grid = comm_grid(shard_elems / 8, 512, max_blocks);
#define SG_RS(F32, ACC, UU) reduce_scatter_fused_kernel<F32, ACC, UU><<<grid, 512, 0, s>>>(bufs, elem_offset, shard_elems, rank, world, scale, out, sumsq_out)
#define SG_RS_U(F32, ACC) do { if (world <= 2) SG_RS(F32, ACC, 4); else if (world <= 4) SG_RS(F32, ACC, 2); else SG_RS(F32, ACC, 1); } while (0)
    if (out_fp32 && accumulate) SG_RS_U(true, true);
    else if (out_fp32) SG_RS_U(true, false);
    else SG_RS_U(false, false);
#undef SG_RS_U
#undef SG_RS
}

void reduce_scatter_multimem(const void* mc_base, size_t elem_offset, size_t shard_elems, int rank, float scale, void* out, int out_fp32,
                             float* sumsq_out, int max_blocks, cudaStream_t s) {
    const int grid = comm_grid(shard_elems / 8, 512, max_blocks);
    if (out_fp32) reduce_scatter_multimem_kernel<true><<<grid, 512, 0, s>>>(mc_base, elem_offset, shard_elems, rank, scale, out, sumsq_out);
    else reduce_scatter_multimem_kernel<false><<<grid, 512, 0, s>>>(mc_base, elem_offset, shard_elems, rank, scale, out, sumsq_out);
}

void all_gather_fused(const PeerPtrs& shards, size_t shard_elem_offset, size_t shard_elems, size_t seg_begin, size_t seg_end, void* out_bf16,
                      void* out_fp8, const float* scale, int max_blocks, cudaStream_t s) {
    if (seg_end <= seg_begin) return;
    const int grid = comm_grid((seg_end - seg_begin) / 8, 512, max_blocks);
    all_gather_fused_kernel<<<grid, 512, 0, s>>>(shards, shard_elem_offset, shard_elems, seg_begin, seg_end, reinterpret_cast<bf16*>(out_bf16),
                                                 reinterpret_cast<uint8_t*>(out_fp8), scale);
}

void all_reduce_small(const PeerPtrs& slots, const PeerPtrs& pads, size_t slot_elem_offset, float* data, int n, int op, int rank, int world,
                      uint32_t epoch, int slot_base, int* error_flag, double budget_s, cudaStream_t s) {
    const long long budget = budget_s > 0 ? static_cast<long long>(budget_s * 2.0e9) : kPeerWaitCycles;
    all_reduce_small_kernel<<<1, 1024, 0, s>>>(slots, pads, slot_elem_offset, data, n, op, rank, world, epoch, slot_base, error_flag, budget);
}

}  // namespace sg

// Launch API of the peer-memory collective kernels (comm_kernels.cu).  Up to 8 ranks on one NVSwitch node.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sg {

constexpr int kMaxPeers = 8;
struct PeerPtrs {
    void* p[kMaxPeers];  // p[r] = base address of rank r's symmetric arena as mapped into THIS process
};

void symm_barrier(const PeerPtrs& pads, int rank, int world, uint32_t epoch, int slot_base, int* error_flag, double budget_s, cudaStream_t s);
void reduce_scatter_fused(const PeerPtrs& bufs, size_t elem_offset, size_t shard_elems, int rank, int world, float scale, void* out, int out_fp32,
                          int accumulate, float* sumsq_out, int max_blocks, cudaStream_t s);
void reduce_scatter_multimem(const void* mc_base, size_t elem_offset, size_t shard_elems, int rank, float scale, void* out, int out_fp32,
                             float* sumsq_out, int max_blocks, cudaStream_t s);
void all_gather_fused(const PeerPtrs& shards, size_t shard_elem_offset, size_t shard_elems, size_t seg_begin, size_t seg_end, void* out_bf16,
                      void* out_fp8, const float* scale, int max_blocks, cudaStream_t s);
void all_reduce_small(const PeerPtrs& slots, const PeerPtrs& pads, size_t slot_elem_offset, float* data, int n, int op, int rank, int world,
                      uint32_t epoch, int slot_base, int* error_flag, double budget_s, cudaStream_t s);

}  // namespace sg

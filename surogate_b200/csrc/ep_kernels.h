// Launch API of the expert-parallel dispatch / combine kernels (ep_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_kernels.h"

namespace sg {

void ep_plan(const PeerPtrs& ctrl, const PeerPtrs& pads, const int* counts, int* offsets, int* dst_base, int* cursors, int E, int rank, int world,
             uint32_t epoch, int slot_base, int capacity_rows, int* error_flag, double budget_s, cudaStream_t s);
void ep_dispatch(const void* x, const int* topk_idx, const float* w, const int* dst_base, const int* row_pos, int* row_map, const PeerPtrs& recv, int tokens,
                 int C, int K, int El, int capacity_rows, int reuse_map, const float* q_scale, float* amax_out, cudaStream_t s);
void ep_row_positions(const int* topk_idx, int* pos, int n_entries, int E, cudaStream_t s);
void ep_combine(const PeerPtrs& outs, const float* w, const int* row_map, void* y, void* rows_out, int tokens, int C, int K, int capacity_rows,
                cudaStream_t s);
void ep_weight_grad(const void* rows, const void* dy, float* d_w, int tokens, int C, int K, cudaStream_t s);

void ep_zero_pad_rows(void* buf, const int* offsets, int El, int C, int capacity_rows, cudaStream_t s);
void copy_rows_upto(const void* src, void* dst, const int* n_rows, int C, int num_sms, cudaStream_t s);

}  // namespace sg

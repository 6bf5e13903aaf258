// Launch API of the MoE routing kernels (moe_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sg {

void moe_softmax_topk(const float* logits, float* topk_w, int* topk_idx, float* probs_out, int* counts, float* prob_sum, float* lse_sq_sum,
                      int tokens, int E, int K, int renorm, int num_sms, cudaStream_t s);
void moe_router_bwd(const float* logits, const int* topk_idx, const float* d_topk_w, const int* counts, const float* d_aux, void* d_logits, int tokens,
                    int E, int K, int renorm, float aux_coef, float z_coef, int num_sms, cudaStream_t s);
void moe_offsets(const int* counts, int* offsets, int* cursors, int E, int capacity_rows, int* error_flag, cudaStream_t s);
void moe_permute(const void* x, const int* topk_idx, const int* offsets, int* cursors, int* row_map, void* xp, int tokens, int C, int K,
                 int expert_base, int num_local, int capacity_rows, cudaStream_t s);
void moe_unpermute(const void* yp, const float* w, const int* row_map, void* y, int tokens, int C, int K, cudaStream_t s);
void moe_unpermute_bwd(const void* dy, const void* yp, const float* w, const int* row_map, void* d_yp, float* d_w, int tokens, int C, int K,
                       cudaStream_t s);

}  // namespace sg

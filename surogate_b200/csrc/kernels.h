// Launch API of the memory-bound kernels in kernels.cu (all pointers are device pointers; bf16 activations).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sg {

void rmsnorm_fwd(const void* x, const void* residual, const void* w, void* res_out, void* y, float* rstd, void* y_fp8, const float* fp8_scale,
                 float* amax, int rows, int C, float eps, cudaStream_t s);
int rmsnorm_bwd_blocks(int rows, int num_sms);
int rmsnorm_bwd_blocks_wide(int rows, int C, int num_sms);
void rmsnorm_bwd_n(const void* dy, const void* x, const void* w, const float* rstd, const void* d_res, void* dx, float* dw_partial, float* dw, int rows,
                   int C, int blocks, cudaStream_t s);
void rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* d_res, void* dx, float* dw_partial, float* dw, int rows,
                 int C, int num_sms, cudaStream_t s);
void swiglu_fwd(const void* x, void* y, void* y_fp8, const float* fp8_scale, float* amax, size_t rows, int M, int num_sms, cudaStream_t s,
                const int* rows_limit = nullptr);
void swiglu_bwd(const void* dy, const void* x, void* dx, size_t rows, int M, int num_sms, cudaStream_t s, const int* rows_limit = nullptr,
                void* dx_fp8 = nullptr, const float* fp8_scale = nullptr, float* amax_out = nullptr);
void zero_empty_groups(void* out, const int* offsets, int groups, size_t bytes_per_group, cudaStream_t s);
void qk_norm_rope_fwd(const void* qkv, const void* qw, const void* kw, const int* pos, void* out, float* q_rstd, float* k_rstd, size_t tokens, int Hq,
                      int Hkv, float eps, float theta, int lim_h, int lim_w, int num_sms, cudaStream_t s);
void qk_norm_rope_bwd(const void* d_out, const void* qkv_pre, const void* qw, const void* kw, const int* pos, void* d_qkv, float* q_rstd,
                      float* k_rstd, float* dqw, float* dkw, size_t tokens, int Hq, int Hkv, float eps, float theta, int lim_h, int lim_w, int num_sms,
                      cudaStream_t s);
void embedding_fwd(const int* tokens, const void* table, void* out, size_t n, int C, int V, int* error_flag, int num_sms, cudaStream_t s);
void embedding_bwd(const int* tokens, const void* d_out, void* d_table, int grad_fp32, size_t n, int C, int num_sms, cudaStream_t s);
void embedding_bwd_sorted(const int* sorted_ids, const long long* order, const void* d_out, void* d_table, int grad_fp32, int n, int C, int V,
                          cudaStream_t s);
void cross_entropy_fwd_bwd(void* logits, const int* targets, float* loss, const float* scale_ptr, float scale_host, int rows, int V, int ld,
                           int write_grad, const float* row_weight, const int* kd_idx, const float* kd_logp, int kd_k, float kd_weight, float* kd_loss,
                           cudaStream_t s);
void quantize_fp8(const void* x, void* q, const float* scale, float* amax, size_t n, int e5m2, int num_sms, cudaStream_t s,
                  const int* rows_limit = nullptr, int row_len = 0);
void amax_bf16(const void* x, float* amax, size_t n, int num_sms, cudaStream_t s, const int* rows_limit = nullptr, int row_len = 0);
void sumsq(const void* x, int is_fp32, float* partial, int nblocks, size_t n, cudaStream_t s);
void adamw_fp32(void* p, int p_fp32, const void* g, int g_fp32, float* m, float* v, const uint8_t* mask, const float* hp, size_t n, int num_sms,
                cudaStream_t s);
void adamw_8bit(void* p, int p_fp32, const void* g, int g_fp32, void* m8, void* v8, void* ms, void* vs, const uint8_t* mask, int block_mask,
                const float* hp, size_t n, int num_sms, cudaStream_t s);

}  // namespace sg

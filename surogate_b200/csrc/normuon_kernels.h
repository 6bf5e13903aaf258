// Launch API of the NorMuon kernels (normuon_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace sg {

void normuon_momentum(const void* g, int g_fp32, void* m, void* u, float* sumsq, const float* hp, float mu, size_t n, int num_sms, cudaStream_t s);
void normuon_momentum8(const void* g, int g_fp32, void* m8, void* ms, void* u, float* sumsq, const float* hp, float mu, size_t n, int num_sms, cudaStream_t s);
void normuon_normalise(void* x, const float* sumsq, size_t n, int num_sms, cudaStream_t s);
void normuon_row_stats(const void* x, float* v, float* sums, const float* hp, float beta2, int R, int C, cudaStream_t s);
void normuon_apply(void* w, int w_fp32, const void* x, const float* v, const float* sums, const float* hp, float update_scale, int cautious, int C,
                   size_t first, size_t count, int num_sms, cudaStream_t s);

}  // namespace sg

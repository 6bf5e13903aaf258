// Launch API of the depth-wise causal convolution kernels (conv1d_kernels.cu).
#pragma once
#include <cuda_runtime.h>

namespace sg {

// x, y: [B, T, C] channels-last (bf16 or fp32, same type); w: fp32 [C, K]; bias: fp32 [C] or null; K <= 4; C % 8 == 0.
// seq_id: int32 [B, T] or null: taps never reach into a position whose id differs (packed documents).
void causal_conv1d_fwd(const void* x, const float* w, const float* bias, const int* seq_id, void* y, int is_fp32, int B, int T, int C, int K, int silu,
                       cudaStream_t s);
// dz: gradient of the convolution output (before any activation).  dw [C, K] and dbias [C] (fp32) are accumulated into.
void causal_conv1d_bwd(const void* dz, const void* x, const float* w, const int* seq_id, void* dx, float* dw, float* dbias, int is_fp32, int B, int T, int C,
                       int K, cudaStream_t s);

}  // namespace sg

// Launch API of the NVFP4 quantisers (nvfp4_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sg {

void nvfp4_quantize_rows(const void* x, void* q, void* sf, const float* amax_tensor, int rows, int K, int stochastic, uint32_t seed, int block2d,
                         int num_sms, cudaStream_t s, int four_over_six = 0);
void nvfp4_quantize_transpose(const void* x, void* q, void* sf, const float* amax_tensor, int R, int C, int stochastic, int hadamard, uint32_t seed,
                              uint32_t sign_mask, cudaStream_t s, int four_over_six = 0);
// four_over_six applies to round-to-nearest quantisation only; its tensors use the encode factor 1536 instead of 2688 (pass it to
// nvfp4_dequantize and use amax / 1536 as the GEMM de-scale)
void nvfp4_dequantize(const void* q, const void* sf, const float* amax_tensor, float amax_div, void* out, int rows, int K, int num_sms, cudaStream_t s,
                      float encode = 2688.f);

}  // namespace sg

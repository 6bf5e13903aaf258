// Launch API of the QLoRA storage dequantisers (qlora_kernels.cu).  n = number of elements (a multiple of 8 and of the block size).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sg {

// absmax (fp32 per block) or, when it is null, the double-quantised triple (int8 codes, fp32 scale per 256 blocks, fp32 offset)
void dequant_nf4(const void* codes, const float* absmax, const int8_t* absmax_q, const float* absmax_scale, const float* absmax_offset, void* out,
                 size_t n, int block, int num_sms, cudaStream_t s);
void dequant_fp8_block(const void* q, const float* scale, void* out, size_t n, int block, int num_sms, cudaStream_t s);
void dequant_nvfp4(const void* codes, const void* sf, const float* ge_inv, void* out, size_t n, int num_sms, cudaStream_t s);
void dequant_mxfp4(const void* codes, const void* scales, void* out, size_t n, int num_sms, cudaStream_t s);

}  // namespace sg

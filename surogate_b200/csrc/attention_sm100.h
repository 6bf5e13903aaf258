// Host API of the tcgen05 flash-attention kernels (attention_sm100.cu).
#pragma once
#include <cuda_runtime.h>

namespace sg {

// qkv: packed [B, T, (Hq + 2*Hkv) * 128] bf16.  out: [B, T, Hq*128] bf16.  lse: [B, T, Hq] fp32 (natural log).
const char* flash_attn_fwd_sm100(const void* qkv, void* out, float* lse, int B, int T, int Hq, int Hkv, float softmax_scale, int* error_flag,
                                 cudaStream_t stream);

// Same contract as flash_attn_fwd_sm100; 128x64 steps and two co-resident CTAs per SM (the default forward).
const char* flash_attn_fwd64_sm100(const void* qkv, void* out, float* lse, int B, int T, int Hq, int Hkv, float softmax_scale, int* error_flag,
                                   cudaStream_t stream, long long* prof = nullptr);

// Backward: d_qkv (same packed layout as qkv) from d_out; `delta` is a [B, T, Hq] fp32 workspace.
const char* flash_attn_bwd_sm100(const void* qkv, const void* out, const void* d_out, const float* lse, float* delta, void* d_qkv, int B, int T, int Hq,
                                 int Hkv, float softmax_scale, int* error_flag, int num_sms, cudaStream_t stream, int variant = 64);

// The two second-generation backward kernels (delta already computed); called by flash_attn_bwd_sm100 unless variant == 128.
const char* flash_attn_bwd64_sm100(const void* qkv, const void* d_out, const float* lse, const float* delta, void* d_qkv, int B, int T, int Hq, int Hkv,
                                   float softmax_scale, int* error_flag, cudaStream_t stream, long long* prof = nullptr);

}  // namespace sg

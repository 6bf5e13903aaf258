// Host API of the tcgen05 flash-attention kernels (attention_fwd64_sm100.cu, attention_bwd64_sm100.cu).
#pragma once
#include <cuda_runtime.h>

namespace sg {

// qkv: packed [B, T, (Hq + 2*Hkv) * 128] bf16.  out: [B, T, Hq*128] bf16.  lse: [B, T, Hq] fp32 (natural log).
// 128 x 64 steps, two co-resident CTAs per SM.  `lo` (optional, [B, T] int32, non-decreasing along each sequence): query t attends
// keys lo[t] <= k <= t: packed documents, sliding windows or both.
const char* flash_attn_fwd64_sm100(const void* qkv, void* out, float* lse, int B, int T, int Hq, int Hkv, float softmax_scale, int* error_flag,
                                   cudaStream_t stream, long long* prof = nullptr, const int* lo = nullptr);

// Backward: d_qkv (same packed layout as qkv) from d_out; `delta` is a [B, T, Hq] fp32 workspace.  With `lo`, `kv_qend` ([B, T/128]
// int32) gives per 128-key tile the exclusive end, in 64-row query tiles, of the queries that can attend it.
const char* flash_attn_bwd_sm100(const void* qkv, const void* out, const void* d_out, const float* lse, float* delta, void* d_qkv, int B, int T, int Hq,
                                 int Hkv, float softmax_scale, int* error_flag, int num_sms, cudaStream_t stream, const int* lo = nullptr,
                                 const int* kv_qend = nullptr);

// The two backward kernels (delta already computed).
const char* flash_attn_bwd64_sm100(const void* qkv, const void* d_out, const float* lse, const float* delta, void* d_qkv, int B, int T, int Hq, int Hkv,
                                   float softmax_scale, int* error_flag, cudaStream_t stream, long long* prof = nullptr, const int* lo = nullptr,
                                   const int* kv_qend = nullptr);

}  // namespace sg

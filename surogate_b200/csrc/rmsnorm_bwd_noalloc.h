// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference implementation.
//
// Who needs it: code that runs where cudaMalloc is off limits — inside a region whose memory footprint was
// fixed in advance (an inference server or a real-time loop that pre-sized every buffer and treats any later
// allocation as a bug), a plug-in embedded in a host application that owns the allocator and hands out no
// memory to guests, or a latency-critical path where an allocation's implicit device synchronisation would
// stall other streams.  Those callers can still provide inputs and outputs; what they cannot provide is the
// per-block partial-sum workspace the kernel needs for the weight gradient.  Here that workspace is a fixed
// array linked into the library image.
//
// Cost and limits
//   * The workspace is SG_NOALLOC_MAX_BLOCKS x SG_NOALLOC_MAX_C floats (160 x 8192 x 4 B = 5 MiB).  Every GPU
//     that loads this library carries it from load until the process exits, whether or not the entry point
//     is ever called.
//   * C (the normalised width) must be a multiple of 8 and at most SG_NOALLOC_MAX_C; larger shapes are refused
//     with SG_NOALLOC_ERR_TOO_LARGE and nothing is launched.
//   * All calls on one GPU share the one workspace.  Two calls that may run at the same time on that GPU
//     (different streams, or different host threads) race on it: serialise them.  The workspace keeps the
//     previous call's contents; the kernels overwrite every element they later read, so no clearing is needed
//     between calls.
//   * The first call on each GPU resolves the workspace's device address (cudaGetSymbolAddress) and reads the
//     SM count; make that first call outside any stream capture.  Later calls only launch kernels.
//     The set-up is safe against several host threads making their first call at once (the record is published with
//     release / acquire ordering under a mutex).
//   * `stream` must belong to the GPU that is current on the calling thread (cudaSetDevice): the workspace address and the
//     block count are those of the current device.
//   * Every data pointer must be 16-byte aligned (the kernels move 16 bytes per lane); otherwise SG_NOALLOC_ERR_BAD_ARGUMENT.
//   * The launch status is read with cudaPeekAtLastError: the thread's CUDA error state is left untouched.  If the thread
//     already carries an unrelated CUDA error, this call reports SG_NOALLOC_ERR_CUDA and the error stays for the caller to read.
//   * The function calls no cudaMalloc / cudaFree and no allocating library routine.
//
// Arguments are raw device pointers with the same meaning and layout as the allocating entry point
// (bf16 [rows, C] activations and gradients, bf16 [C] weight, fp32 [rows] rstd, optional bf16 [rows, C]
// residual-stream gradient that is added to dx, fp32 [C] dw).  Returns 0 on success.
#pragma once
#include <cuda_runtime.h>

#define SG_NOALLOC_MAX_BLOCKS 160
#define SG_NOALLOC_MAX_C 8192

#define SG_NOALLOC_OK 0
#define SG_NOALLOC_ERR_BAD_ARGUMENT 1
#define SG_NOALLOC_ERR_TOO_LARGE 2
#define SG_NOALLOC_ERR_CUDA 3

#ifdef __cplusplus
extern "C" {
#endif

int sg_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* d_res, void* dx, float* dw, int rows,
                           int C, cudaStream_t stream);

// Human-readable text for a return code of sg_rmsnorm_bwd_noalloc (static storage; never NULL).
const char* sg_rmsnorm_bwd_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif

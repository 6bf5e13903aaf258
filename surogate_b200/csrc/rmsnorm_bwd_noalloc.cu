// Allocation-free RMSNorm backward: the same kernels as sg::rmsnorm_bwd, with the partial-sum workspace taken
// from a fixed array in the library image instead of from the caller.  See rmsnorm_bwd_noalloc.h for the
// contract (limits, sharing, first-call set-up).
#include "rmsnorm_bwd_noalloc.h"

#include <atomic>
#include <cstdint>
#include <mutex>

#include "kernels.h"

namespace {

// Per-block partial sums of the weight gradient: [blocks <= SG_NOALLOC_MAX_BLOCKS][C <= SG_NOALLOC_MAX_C] floats.
// In host code this name is only a handle for the symbol, not an address a kernel can use; the device address
// is looked up once per GPU below.
static __device__ __align__(256) float g_dw_partial_workspace[SG_NOALLOC_MAX_BLOCKS * SG_NOALLOC_MAX_C];

constexpr int kMaxDevices = 64;

// Per-GPU set-up record, published with release / acquire ordering: a host thread that sees `ready` also sees the address and the
// SM count written before it.  Two threads that race through the first call both resolve the same values; the stores are idempotent.
struct DeviceSetup {
    std::atomic<int> ready{0};
    float* workspace = nullptr;
    int sm_count = 0;
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

// First use on the current GPU: resolve the workspace's device address and the SM count.
int setup_current_device(int* device_out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SG_NOALLOC_ERR_CUDA;
    DeviceSetup& st = g_setup[dev];
    if (st.ready.load(std::memory_order_acquire) == 0) {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (st.ready.load(std::memory_order_relaxed) == 0) {
            float* ptr = nullptr;
            if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_dw_partial_workspace) != cudaSuccess || ptr == nullptr) return SG_NOALLOC_ERR_CUDA;
            int sms = 0;
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return SG_NOALLOC_ERR_CUDA;
            st.workspace = ptr;
            st.sm_count = sms;
            st.ready.store(1, std::memory_order_release);
        }
    }
    *device_out = dev;
    return SG_NOALLOC_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int sg_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* d_res, void* dx, float* dw,
                                      int rows, int C, cudaStream_t stream) {
    if (!dy || !x || !w || !rstd || !dx || !dw || rows <= 0 || C <= 0 || (C % 8) != 0) return SG_NOALLOC_ERR_BAD_ARGUMENT;
    // the kernels read and write 16 bytes at a time (8 bf16 / 4 floats per lane)
    if (!aligned16(dy) || !aligned16(x) || !aligned16(w) || !aligned16(dx) || !aligned16(dw) || (d_res && !aligned16(d_res))) return SG_NOALLOC_ERR_BAD_ARGUMENT;
    if (C > SG_NOALLOC_MAX_C) return SG_NOALLOC_ERR_TOO_LARGE;
    int dev = -1;
    const int rc = setup_current_device(&dev);
    if (rc != SG_NOALLOC_OK) return rc;
    // The launcher uses min(rows, 2 * sms) blocks; cap the SM count it sees so the block count fits the workspace.
    int sms = g_setup[dev].sm_count;
    if (2 * sms > SG_NOALLOC_MAX_BLOCKS) sms = SG_NOALLOC_MAX_BLOCKS / 2;
    if (sg::rmsnorm_bwd_blocks(rows, sms) > SG_NOALLOC_MAX_BLOCKS) return SG_NOALLOC_ERR_TOO_LARGE;
    sg::rmsnorm_bwd(dy, x, w, rstd, d_res, dx, g_setup[dev].workspace, dw, rows, C, sms, stream);
    // Peek, not get: the calling thread's CUDA error state is reported but left as it is, so an earlier error of the caller's own
    // is neither cleared nor hidden from the caller's next check (it does make this call report failure).
    return cudaPeekAtLastError() == cudaSuccess ? SG_NOALLOC_OK : SG_NOALLOC_ERR_CUDA;
}

extern "C" const char* sg_rmsnorm_bwd_noalloc_strerror(int code) {
    switch (code) {
        case SG_NOALLOC_OK: return "success";
        case SG_NOALLOC_ERR_BAD_ARGUMENT: return "bad argument: null pointer, pointer not 16-byte aligned, non-positive size, or C not a multiple of 8";
        case SG_NOALLOC_ERR_TOO_LARGE: return "shape exceeds the built-in workspace (C must be <= 8192)";
        case SG_NOALLOC_ERR_CUDA: return "a CUDA runtime call failed (device query, symbol lookup or kernel launch), or the calling thread already had a CUDA error pending";
        default: return "unknown error code";
    }
}

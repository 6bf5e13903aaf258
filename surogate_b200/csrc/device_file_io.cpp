// File -> device-memory reads for checkpoint loading.
//
// Two routes, chosen per call:
//   * GPUDirect Storage: libcufile is opened at run time (dlopen; no link-time dependency), the file is opened with O_DIRECT
//     and cuFileRead moves the bytes from the drive into device memory without a bounce through host memory.  Any failure on the
//     way (library missing, driver not open, handle not registrable, short read) falls back to the staged route for this call.
//   * staged: pread into two pinned staging buffers and cudaMemcpyAsync from them, so the disk read of chunk k+1 overlaps the
//     host-to-device copy of chunk k.
// Reference counterpart: csrc/src/utilities/cu_file.cpp (cuFile reads with a run-time fallback to buffered I/O).
#include <cuda_runtime.h>
#include <cufile.h>
#include <dlfcn.h>
#include <fcntl.h>
#include <torch/extension.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <mutex>
#include <string>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

namespace {

using torch::Tensor;

struct CuFileApi {
    void* lib = nullptr;
    CUfileError_t (*driver_open)() = nullptr;
    CUfileError_t (*handle_register)(CUfileHandle_t*, CUfileDescr_t*) = nullptr;
    void (*handle_deregister)(CUfileHandle_t) = nullptr;
    ssize_t (*read)(CUfileHandle_t, void*, size_t, off_t, off_t) = nullptr;
    bool driver_ok = false;
    std::string why;
};

CuFileApi& cufile_api() {
    static CuFileApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        for (const char* name : {"libcufile.so.0", "libcufile.so"}) {
            api.lib = dlopen(name, RTLD_NOW | RTLD_LOCAL);
            if (api.lib) break;
        }
        if (!api.lib) {
            api.why = "libcufile not found";
            return;
        }
        api.driver_open = reinterpret_cast<decltype(api.driver_open)>(dlsym(api.lib, "cuFileDriverOpen"));
        api.handle_register = reinterpret_cast<decltype(api.handle_register)>(dlsym(api.lib, "cuFileHandleRegister"));
        api.handle_deregister = reinterpret_cast<decltype(api.handle_deregister)>(dlsym(api.lib, "cuFileHandleDeregister"));
        api.read = reinterpret_cast<decltype(api.read)>(dlsym(api.lib, "cuFileRead"));
        if (!api.driver_open || !api.handle_register || !api.handle_deregister || !api.read) {
            api.why = "libcufile lacks a needed symbol";
            return;
        }
        const CUfileError_t st = api.driver_open();
        if (st.err != CU_FILE_SUCCESS) {
            api.why = "cuFileDriverOpen failed (" + std::to_string(static_cast<int>(st.err)) + ")";
            return;
        }
        api.driver_ok = true;
    });
    return api;
}

// true when all bytes arrived through cuFile; false (with `why`) when the caller should use the staged route
bool read_gds(const std::string& path, uint64_t file_offset, uint64_t nbytes, void* dst, std::string& why) {
    CuFileApi& api = cufile_api();
    if (!api.driver_ok) {
        why = api.why;
        return false;
    }
    const int fd = open(path.c_str(), O_RDONLY | O_DIRECT);
    if (fd < 0) {
        why = std::string("open(O_DIRECT): ") + std::strerror(errno);
        return false;
    }
    CUfileDescr_t descr;
    std::memset(&descr, 0, sizeof(descr));
    descr.handle.fd = fd;
    descr.type = CU_FILE_HANDLE_TYPE_OPAQUE_FD;
    CUfileHandle_t handle;
    const CUfileError_t st = api.handle_register(&handle, &descr);
    if (st.err != CU_FILE_SUCCESS) {
        close(fd);
        why = "cuFileHandleRegister failed (" + std::to_string(static_cast<int>(st.err)) + ")";
        return false;
    }
    bool ok = true;
    uint64_t done = 0;
    while (done < nbytes) {
        const size_t want = static_cast<size_t>(std::min<uint64_t>(nbytes - done, 1ull << 30));
        const ssize_t got = api.read(handle, dst, want, static_cast<off_t>(file_offset + done), static_cast<off_t>(done));
        if (got <= 0) {
            why = "cuFileRead returned " + std::to_string(static_cast<long long>(got));
            ok = false;
            break;
        }
        done += static_cast<uint64_t>(got);
    }
    api.handle_deregister(handle);
    close(fd);
    return ok;
}

struct Staging {
    void* buf[2] = {nullptr, nullptr};
    cudaEvent_t free_ev[2] = {nullptr, nullptr};
    size_t bytes = 0;
    ~Staging() {
        for (int i = 0; i < 2; ++i) {
            if (buf[i]) cudaFreeHost(buf[i]);
            if (free_ev[i]) cudaEventDestroy(free_ev[i]);
        }
    }
};

void read_staged(const std::string& path, uint64_t file_offset, uint64_t nbytes, char* dst, cudaStream_t stream) {
    constexpr size_t CHUNK = 32u << 20;
    Staging st;
    st.bytes = static_cast<size_t>(std::min<uint64_t>(CHUNK, std::max<uint64_t>(nbytes, 1)));
    for (int i = 0; i < 2; ++i) {
        TORCH_CHECK(cudaHostAlloc(&st.buf[i], st.bytes, cudaHostAllocDefault) == cudaSuccess, "pinned staging buffer allocation failed");
        TORCH_CHECK(cudaEventCreateWithFlags(&st.free_ev[i], cudaEventDisableTiming) == cudaSuccess, "event creation failed");
    }
    const int fd = open(path.c_str(), O_RDONLY);
    TORCH_CHECK(fd >= 0, "cannot open ", path, ": ", std::strerror(errno));
    uint64_t done = 0;
    int k = 0;
    bool used[2] = {false, false};
    std::string err;
    while (done < nbytes && err.empty()) {
        const size_t want = static_cast<size_t>(std::min<uint64_t>(nbytes - done, st.bytes));
        if (used[k] && cudaEventSynchronize(st.free_ev[k]) != cudaSuccess) {
            err = "waiting for a staging buffer failed";
            break;
        }
        size_t got = 0;
        while (got < want) {
            const ssize_t r = pread(fd, static_cast<char*>(st.buf[k]) + got, want - got, static_cast<off_t>(file_offset + done + got));
            if (r < 0 && errno == EINTR) continue;
            if (r <= 0) {
                err = r == 0 ? "unexpected end of file" : std::string("pread: ") + std::strerror(errno);
                break;
            }
            got += static_cast<size_t>(r);
        }
        if (!err.empty()) break;
        if (cudaMemcpyAsync(dst + done, st.buf[k], want, cudaMemcpyHostToDevice, stream) != cudaSuccess || cudaEventRecord(st.free_ev[k], stream) != cudaSuccess) {
            err = "host-to-device copy failed";
            break;
        }
        used[k] = true;
        done += want;
        k ^= 1;
    }
    close(fd);
    cudaStreamSynchronize(stream);  // the staging buffers are freed on return
    TORCH_CHECK(err.empty(), path, ": ", err);
}

// dst: contiguous CUDA tensor of at least nbytes.  Returns "gds" or "staged" (+ the reason GDS was not used).
std::string read_file_to_device(const std::string& path, uint64_t file_offset, uint64_t nbytes, Tensor dst, bool try_gds) {
    TORCH_CHECK(dst.is_cuda() && dst.is_contiguous(), "destination must be a contiguous CUDA tensor");
    TORCH_CHECK(static_cast<uint64_t>(dst.numel()) * dst.element_size() >= nbytes, "destination is smaller than the requested range");
    const c10::cuda::CUDAGuard guard(dst.device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
    std::string why;
    if (try_gds) {
        TORCH_CHECK(cudaStreamSynchronize(stream) == cudaSuccess, "stream synchronize failed");  // cuFileRead is not stream-ordered
        if (read_gds(path, file_offset, nbytes, dst.data_ptr(), why)) return "gds";
    }
    {
        pybind11::gil_scoped_release rel;
        read_staged(path, file_offset, nbytes, static_cast<char*>(dst.data_ptr()), stream);
    }
    return why.empty() ? "staged" : "staged (" + why + ")";
}

}  // namespace

void sg_register_device_io(pybind11::module_& m) {
    m.def("read_file_to_device", &read_file_to_device, pybind11::arg("path"), pybind11::arg("file_offset"), pybind11::arg("nbytes"), pybind11::arg("dst"),
          pybind11::arg("try_gds") = false,
          "Read a byte range of a file into a CUDA tensor: GPUDirect Storage when asked for and available, else pinned double-buffered staging.");
}

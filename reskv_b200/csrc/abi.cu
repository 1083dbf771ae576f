// Error reporting and device queries shared by every entry point.
#include <cstring>

#include "common.cuh"

namespace reskv {
namespace {
thread_local char g_error[512] = "";
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return RESKV_OK;
    return fail(RESKV_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

int check_device_pointer(const void* ptr, const char* who, const char* what) {
    cudaPointerAttributes attr{};
    const cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
    if (e != cudaSuccess) {
        cudaGetLastError();  // the failed query must not poison later calls
        return fail(RESKV_ERR_INVALID, "%s: %s is not memory a CUDA device can be asked about (%s)", who, what,
                    cudaGetErrorString(e));
    }
    if (attr.type == cudaMemoryTypeManaged) return RESKV_OK;
    if (attr.type != cudaMemoryTypeDevice)
        return fail(RESKV_ERR_INVALID, "%s: %s must be device memory, got a host pointer", who, what);
    int dev = -1;
    if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    if (attr.device != dev)
        return fail(RESKV_ERR_INVALID,
                    "%s: %s lives on device %d but device %d is current; make the tensors' device current "
                    "(cudaSetDevice) before the call",
                    who, what, attr.device, dev);
    return RESKV_OK;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}
}  // namespace reskv

extern "C" const char* reskv_last_error(void) { return reskv::g_error; }

extern "C" int reskv_version(void) { return 100; }

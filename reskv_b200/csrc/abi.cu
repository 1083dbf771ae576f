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

// Shared device/host helpers for the sm_100a kernels of the compressed-KV path.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/reskv_b200.h"

namespace reskv {

constexpr int kHeadDim = 128;
constexpr int kMaxClusters = 64;

// ---- host side: error reporting ---------------------------------------------
// Every entry point returns 0 or a negative RESKV_ERR_* code and leaves a
// message for reskv_last_error() (thread local).
int fail(int code, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Every entry point launches on the CURRENT device (as the stream it is given must belong to it): `ptr` has to be
// memory of that device (or managed memory).  A host pointer or another GPU's memory is refused with
// RESKV_ERR_INVALID before anything is launched -- a kernel given such a pointer would fault.
int check_device_pointer(const void* ptr, const char* who, const char* what);

// Number of SMs of the current device (cached per device).
int sm_count();

// ---- device side: async bulk copies (TMA, 1-D) and mbarriers -------------------
// All waits are bounded: a wait that runs out records RESKV_STATUS_WAIT_TIMEOUT in
// the kernel's status word and returns, so a lost copy can never hang the GPU.

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

// Makes freshly initialised barriers visible to the async proxy.
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the limit ran out (about a second of
// polling); the caller records the failure and carries on without the data.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// 16-byte asynchronous copy global -> shared of the calling thread (both addresses 16-byte aligned).
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}

// One arrival on `bar` once all earlier cp_async16 copies of the calling thread have landed.  The
// arrival is not added to the barrier's pending count: the barrier's initial count includes it.
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

}  // namespace reskv

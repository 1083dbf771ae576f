// Device-resident decode-step state and the dense-window append that goes with it.
//
// A decode step of a model touches, per layer, the dense window (append the new token) and the
// fused attention (query position, number of window tokens).  When those two numbers live in
// device memory -- step_state = {query position, window tokens} -- the whole step can be captured
// in one CUDA graph and replayed: the append and the decode kernels read them, and one tiny kernel
// advances them at the end of the step.
#include "common.cuh"

namespace reskv {
namespace {

// grid = units, block = 128 threads: copy the new token's rotated key, raw key and value rows
// into the last counted slot, step_state[1] - 1, of every unit's window (the caller advances the
// window count first, so that the attention of the same step already sees the new token).
__global__ void window_append_kernel(__half* win_k, __half* win_raw, __half* win_v, const __half* k_rot,
                                     const __half* k_raw, const __half* v, int capacity,
                                     const int32_t* __restrict__ step_state) {
    const int unit = blockIdx.x, d = threadIdx.x;
    const int slot = min(max(step_state[1] - 1, 0), capacity - 1);
    const size_t dst = (static_cast<size_t>(unit) * capacity + slot) * kHeadDim + d;
    const size_t src = static_cast<size_t>(unit) * kHeadDim + d;
    win_k[dst] = k_rot[src];
    win_raw[dst] = k_raw[src];
    win_v[dst] = v[src];
}

// Same copy with the slot given by the host (eager callers that track the window length themselves).
__global__ void window_write_kernel(__half* win_k, __half* win_raw, __half* win_v, const __half* k_rot,
                                    const __half* k_raw, const __half* v, int capacity, int slot) {
    const int unit = blockIdx.x, d = threadIdx.x;
    const size_t dst = (static_cast<size_t>(unit) * capacity + slot) * kHeadDim + d;
    const size_t src = static_cast<size_t>(unit) * kHeadDim + d;
    win_k[dst] = k_rot[src];
    win_raw[dst] = k_raw[src];
    win_v[dst] = v[src];
}

__global__ void step_advance_kernel(int32_t* step_state, int pos_inc, int live_inc) {
    if (threadIdx.x == 0) {
        step_state[0] += pos_inc;
        step_state[1] += live_inc;
    }
}

}  // namespace
}  // namespace reskv

using namespace reskv;

extern "C" int reskv_window_append(void* window_k, void* window_raw, void* window_v, const void* k_rot,
                                   const void* k_raw, const void* v, int batch, int kv_heads, int window_capacity,
                                   const int32_t* step_state, void* stream) {
    if (!window_k || !window_raw || !window_v || !k_rot || !k_raw || !v || !step_state)
        return fail(RESKV_ERR_INVALID, "window_append: null pointer");
    if (batch < 1 || kv_heads < 1 || window_capacity < 1)
        return fail(RESKV_ERR_INVALID, "window_append: batch, heads and capacity must be positive");
    window_append_kernel<<<batch * kv_heads, kHeadDim, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__half*>(window_k), static_cast<__half*>(window_raw), static_cast<__half*>(window_v),
        static_cast<const __half*>(k_rot), static_cast<const __half*>(k_raw), static_cast<const __half*>(v),
        window_capacity, step_state);
    return check_cuda(cudaGetLastError(), "window_append launch");
}

extern "C" int reskv_window_write(void* window_k, void* window_raw, void* window_v, const void* k_rot,
                                  const void* k_raw, const void* v, int batch, int kv_heads, int window_capacity,
                                  int slot, void* stream) {
    if (!window_k || !window_raw || !window_v || !k_rot || !k_raw || !v)
        return fail(RESKV_ERR_INVALID, "window_write: null pointer");
    if (batch < 1 || kv_heads < 1 || window_capacity < 1)
        return fail(RESKV_ERR_INVALID, "window_write: batch, heads and capacity must be positive");
    if (slot < 0 || slot >= window_capacity)
        return fail(RESKV_ERR_INVALID, "window_write: slot %d outside the window of %d tokens", slot, window_capacity);
    if (int rc = check_device_pointer(window_k, "window_write", "window_k")) return rc;
    window_write_kernel<<<batch * kv_heads, kHeadDim, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__half*>(window_k), static_cast<__half*>(window_raw), static_cast<__half*>(window_v),
        static_cast<const __half*>(k_rot), static_cast<const __half*>(k_raw), static_cast<const __half*>(v),
        window_capacity, slot);
    return check_cuda(cudaGetLastError(), "window_write launch");
}

extern "C" int reskv_step_advance(int32_t* step_state, int position_increment, int window_increment, void* stream) {
    if (!step_state) return fail(RESKV_ERR_INVALID, "step_advance: null step state");
    step_advance_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(step_state, position_increment,
                                                                        window_increment);
    return check_cuda(cudaGetLastError(), "step_advance launch");
}

// Small fused kernels of a decoder layer's decode step around the attention call: RMS norm,
// "split the fused QKV projection, rotate, append to the dense window", and SiLU(gate) * up.
//
// A decode step is launch-bound at small batch: in plain tensor ops these three pieces are ~30
// launches per layer, here they are three.  All of them read the decode position / window count
// from the device-side step state, so they can sit in the same captured graph as the attention.
#include "common.cuh"

namespace reskv {
namespace {

constexpr int kNormThreads = 256;

// one CTA per row: out = fp16( fp32(x) * rsqrt(mean(x^2) + eps) * fp32(w) )
__global__ void __launch_bounds__(kNormThreads) rms_norm_kernel(const __half* __restrict__ x, const __half* __restrict__ w,
                                                                __half* __restrict__ out, int dim, float eps) {
    __shared__ float part[kNormThreads / 32];
    const size_t row = blockIdx.x;
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    uint4* orow = reinterpret_cast<uint4*>(out + row * dim);
    const int chunks = dim / 8;
    float acc = 0.f;
    for (int c = threadIdx.x; c < chunks; c += kNormThreads) {
        const uint4 v = xr[c];
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            acc = fmaf(f.x, f.x, acc);
            acc = fmaf(f.y, f.y, acc);
        }
    }
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < kNormThreads / 32; ++i) total += part[i];
    const float inv = rsqrtf(total / static_cast<float>(dim) + eps);
    for (int c = threadIdx.x; c < chunks; c += kNormThreads) {
        const uint4 v = xr[c], g = wr[c];
        const __half2* h = reinterpret_cast<const __half2*>(&v);
        const __half2* gh = reinterpret_cast<const __half2*>(&g);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]), gw = __half22float2(gh[i]);
            oh[i] = __floats2half2_rn(f.x * inv * gw.x, f.y * inv * gw.y);
        }
        orow[c] = o;
    }
}

// grid (q_heads + 2 kv_heads, batch), 64 threads: thread i owns the RoPE pair (i, i + 64) of one
// head of the fused projection row [q heads | k heads | v heads].  Position = step_state[0].
__global__ void __launch_bounds__(64) rope_split_kernel(const __half* __restrict__ qkv, int q_heads, int kv_heads,
                                                        const float* __restrict__ inv_freq,
                                                        const int32_t* __restrict__ step_state, __half* q_raw,
                                                        __half* q_rot, __half* k_rot, __half* v_out, __half* win_k,
                                                        __half* win_raw, __half* win_v, int capacity) {
    const int head = blockIdx.x, b = blockIdx.y, i = threadIdx.x;
    const int heads = q_heads + 2 * kv_heads;
    const __half* src = qkv + (static_cast<size_t>(b) * heads + head) * kHeadDim;
    const __half lo = src[i], hi = src[i + 64];
    if (head >= q_heads + kv_heads) {  // value head: copy
        const int h = head - q_heads - kv_heads;
        const size_t unit = static_cast<size_t>(b) * kv_heads + h;
        if (v_out) v_out[unit * kHeadDim + i] = lo, v_out[unit * kHeadDim + i + 64] = hi;
        if (win_v) {
            const int slot = min(max(step_state[1] - 1, 0), capacity - 1);
            __half* dst = win_v + (unit * capacity + slot) * kHeadDim;
            dst[i] = lo, dst[i + 64] = hi;
        }
        return;
    }
    float s, c;
    sincosf(static_cast<float>(step_state[0]) * inv_freq[i], &s, &c);
    const float a = __half2float(lo), bb = __half2float(hi);
    const __half rlo = __float2half_rn(a * c - bb * s), rhi = __float2half_rn(bb * c + a * s);
    if (head < q_heads) {
        const size_t row = (static_cast<size_t>(b) * q_heads + head) * kHeadDim;
        if (q_raw) q_raw[row + i] = lo, q_raw[row + i + 64] = hi;
        q_rot[row + i] = rlo, q_rot[row + i + 64] = rhi;
        return;
    }
    const int h = head - q_heads;
    const size_t unit = static_cast<size_t>(b) * kv_heads + h;
    if (k_rot) k_rot[unit * kHeadDim + i] = rlo, k_rot[unit * kHeadDim + i + 64] = rhi;
    if (win_k) {
        const int slot = min(max(step_state[1] - 1, 0), capacity - 1);
        __half* dk = win_k + (unit * capacity + slot) * kHeadDim;
        __half* dr = win_raw + (unit * capacity + slot) * kHeadDim;
        dk[i] = rlo, dk[i + 64] = rhi;
        dr[i] = lo, dr[i + 64] = hi;
    }
}

// out[r][j] = fp16( fp16(silu(gate[r][j])) * up[r][j] ), gate_up = [rows, gate | up]
__global__ void silu_mul_kernel(const __half* __restrict__ gate_up, __half* __restrict__ out, int ffn, long long total) {
    const long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 2;
    if (idx >= total) return;
    const long long r = idx / ffn;
    const int j = static_cast<int>(idx % ffn);
    const __half2 g = *reinterpret_cast<const __half2*>(gate_up + r * 2 * ffn + j);
    const __half2 u = *reinterpret_cast<const __half2*>(gate_up + r * 2 * ffn + ffn + j);
    const float2 gf = __half22float2(g), uf = __half22float2(u);
    const __half2 act = __floats2half2_rn(gf.x / (1.f + expf(-gf.x)), gf.y / (1.f + expf(-gf.y)));
    const float2 af = __half22float2(act);
    *reinterpret_cast<__half2*>(out + idx) = __floats2half2_rn(af.x * uf.x, af.y * uf.y);
}

}  // namespace
}  // namespace reskv

using namespace reskv;

extern "C" int reskv_rms_norm(const void* x, const void* weight, void* out, int rows, int dim, float eps, void* stream) {
    if (!x || !weight || !out) return fail(RESKV_ERR_INVALID, "rms_norm: null pointer");
    if (rows < 1 || dim < 8 || dim % 8) return fail(RESKV_ERR_INVALID, "rms_norm: rows must be positive and dim a positive multiple of 8");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(RESKV_ERR_INVALID, "rms_norm: pointers must be 16-byte aligned");
    rms_norm_kernel<<<rows, kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), static_cast<const __half*>(weight), static_cast<__half*>(out), dim, eps);
    return check_cuda(cudaGetLastError(), "rms_norm launch");
}

extern "C" int reskv_rope_split(const void* qkv, int batch, int q_heads, int kv_heads, const float* inv_freq,
                                const int32_t* step_state, void* q_raw, void* q_rot, void* k_rot, void* v_out,
                                void* window_k, void* window_raw, void* window_v, int window_capacity, void* stream) {
    if (!qkv || !inv_freq || !step_state || !q_rot) return fail(RESKV_ERR_INVALID, "rope_split: null pointer");
    if (batch < 1 || q_heads < 1 || kv_heads < 1) return fail(RESKV_ERR_INVALID, "rope_split: batch and head counts must be positive");
    const bool window = window_k || window_raw || window_v;
    if (window && (!window_k || !window_raw || !window_v || window_capacity < 1))
        return fail(RESKV_ERR_INVALID, "rope_split: a window needs its three buffers and a positive capacity");
    if (!window && (!k_rot || !v_out)) return fail(RESKV_ERR_INVALID, "rope_split: nowhere to write keys and values");
    const dim3 grid(q_heads + 2 * kv_heads, batch);
    rope_split_kernel<<<grid, 64, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(qkv), q_heads, kv_heads, inv_freq, step_state, static_cast<__half*>(q_raw),
        static_cast<__half*>(q_rot), static_cast<__half*>(k_rot), static_cast<__half*>(v_out),
        static_cast<__half*>(window_k), static_cast<__half*>(window_raw), static_cast<__half*>(window_v), window_capacity);
    return check_cuda(cudaGetLastError(), "rope_split launch");
}

extern "C" int reskv_silu_mul(const void* gate_up, void* out, int rows, int ffn, void* stream) {
    if (!gate_up || !out) return fail(RESKV_ERR_INVALID, "silu_mul: null pointer");
    if (rows < 1 || ffn < 2 || ffn % 2) return fail(RESKV_ERR_INVALID, "silu_mul: rows must be positive and ffn a positive even number");
    const long long total = static_cast<long long>(rows) * ffn;
    const int threads = 256;
    const long long blocks = (total / 2 + threads - 1) / threads;
    silu_mul_kernel<<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(gate_up), static_cast<__half*>(out), ffn, total);
    return check_cuda(cudaGetLastError(), "silu_mul launch");
}

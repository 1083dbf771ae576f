// Definitions shared by the residual packers (compress_topk.cu: one thread per token, the form every layout of
// the reference uses when its pointers are 16-byte aligned; compress.cu: one warp per token, the compact layout
// and the route for unaligned pointers).
#pragma once

#include "common.cuh"

namespace reskv {

struct EncodeParams {
    const __half* x;        // [units, x_stride, 128]
    const __half* cen;      // [units, clusters, 128]
    const int32_t* ids;     // [units, tokens]
    void* payload;          // layout dependent
    void* meta;             // layout dependent or null
    __half* scale;          // [units, out_stride] or null
    int64_t x_stride, out_stride;
    int units, tokens, clusters, nnz;
};

// Launchers of the thread-per-token kernels (compress_topk.cu).
int launch_topk_bitmap_fp16(const EncodeParams& p, cudaStream_t stream);
int launch_topk_quantized(const EncodeParams& p, int bits, cudaStream_t stream);
int launch_topk_tiled_fp16(const EncodeParams& p, bool indexed, cudaStream_t stream);  // tile masks / 4:16 indices
int launch_topk_structured_int4(const EncodeParams& p, cudaStream_t stream);

namespace {

constexpr int kWarpsPerCta = 8;
constexpr uint32_t kFull = 0xffffffffu;


// The reference is built with --use_fast_math: `a / b` is the GPU's approximate division (one reciprocal
// approximation times the numerator, div.approx.ftz.f32) and a division by a constant becomes a multiplication
// by its rounded reciprocal.  Quantised codes whose exact quotient sits on a rounding boundary depend on that,
// so the same instruction is issued here (vectors recorded from the reference's kernels on a B200 are matched
// to the bit, including the tokens whose scale underflows to 0).
__device__ __forceinline__ float div_fast(float a, float b) {
    float q;
    asm("div.approx.ftz.f32 %0, %1, %2;" : "=f"(q) : "f"(a), "f"(b));
    return q;
}

// (int)lrintf(x): round to nearest even into 64 bits (saturating; NaN -> INT64_MIN), keep the low 32 bits.
// Finite quotients are unaffected; +inf becomes -1 and -inf / NaN become 0, which is what the reference's
// `(int)lrintf(r / 0)` yields for a token whose FP16 scale underflowed (compression.cu:366-367).
__device__ __forceinline__ int lrint_low32(float x) { return static_cast<int>(__float2ll_rn(x)); }

// Scale of the unstructured quantiser: fp16(amax / QMAX) with the division by the constant done as a
// multiplication by fp32(1 / QMAX) (compression.cu:354-355 under --use_fast_math); 1 for an all-zero selection.
template <int QMAX>
__device__ __forceinline__ __half quant_scale(float amax) {
    constexpr float kRecip = 1.0f / static_cast<float>(QMAX);
    return amax > 0.f ? __float2half_rn(amax * kRecip) : __float2half_rn(1.f);
}

template <int QMAX>
__device__ __forceinline__ int quant_code(float r, float s) {
    return max(-QMAX, min(QMAX, lrint_low32(div_fast(r, s))));
}

}  // namespace
}  // namespace reskv

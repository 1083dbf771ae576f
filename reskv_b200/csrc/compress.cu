// Residual packers: x - centroid[id] -> top-magnitude selection -> packed layout.
// This file holds the C entry points of all layouts and the kernel of the compact quantised layout; the
// layouts of the reference run one thread per token and live in compress_topk.cu.
//
// Compact layout: one warp encodes one token; lane l owns coordinates {l, l+32, l+64, l+96}.
// With that ownership a warp vote of "lane keeps coordinate l+32i" *is* the
// keep-mask of coordinates 32i..32i+31 (LSB = lowest coordinate), and ranks are
// popcounts of votes.  Rounding points (they decide bit-exactness against the
// reference): r = fp32(x) - fp32(c); the selection key is |fp16(r)|;
// quantisers divide the FP32 r with the GPU's approximate
// division, as the reference's fast-math build does (see div_fast).
// Ties keep the lower coordinate.
//
// The global top-k is a bisection on the 15-bit key
// pattern: a vote per owned coordinate counts the keys >= candidate, so no data
// moves between lanes.
#include "compress_common.cuh"

namespace reskv {
namespace {

struct Residual {
    float r[4];       // fp32 residual of coordinates lane + 32 i
    uint32_t key[4];  // bit pattern of |fp16(r)|, monotone in magnitude
    __half h[4];      // fp16(r)
};

__device__ __forceinline__ Residual load_residual(const EncodeParams& p, int unit, int t, int lane) {
    const __half* xr = p.x + (static_cast<size_t>(unit) * p.x_stride + t) * kHeadDim;
    int id = p.ids[static_cast<size_t>(unit) * p.tokens + t];
    id = min(max(id, 0), p.clusters - 1);
    const __half* cr = p.cen + (static_cast<size_t>(unit) * p.clusters + id) * kHeadDim;
    Residual out;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float r = __half2float(xr[lane + 32 * i]) - __half2float(__ldg(cr + lane + 32 * i));
        out.r[i] = r;
        out.h[i] = __float2half_rn(r);
        out.key[i] = __half_as_ushort(out.h[i]) & 0x7fffu;
    }
    return out;
}

// keep[i] = coordinate lane+32i is among the `k` largest keys of the token,
// lower coordinate first among equal keys.  vote[i] = warp mask of keep[i].
__device__ __forceinline__ void select_topk(const uint32_t (&key)[4], int k, int lane, bool (&keep)[4],
                                            uint32_t (&vote)[4]) {
    // largest v with count(key >= v) >= k
    uint32_t v = 0;
#pragma unroll
    for (int bit = 14; bit >= 0; --bit) {
        const uint32_t cand = v | (1u << bit);
        int mine = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) mine += key[i] >= cand;
        if (__reduce_add_sync(kFull, mine) >= k) v = cand;
    }
    int above = 0;
    uint32_t eq[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        above += __popc(__ballot_sync(kFull, key[i] > v));
        eq[i] = __ballot_sync(kFull, key[i] == v);
    }
    const int need = k - above;  // how many of the keys equal to v are kept
    const uint32_t below = (1u << lane) - 1u;
    int before = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        keep[i] = key[i] > v || (key[i] == v && before + __popc(eq[i] & below) < need);
        before += __popc(eq[i]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) vote[i] = __ballot_sync(kFull, keep[i]);
}

// ---- compact quantised: bitmap + codes of the retained coordinates only ---------------
// Same selection, scale and codes as encode_quantized_kernel; code of rank r (ascending
// coordinate) at bit (r % kPer) * BITS of word r / kPer.
template <int BITS>
__global__ void __launch_bounds__(kWarpsPerCta * 32) encode_compact_kernel(const EncodeParams p) {
    constexpr int kQmax = (1 << (BITS - 1)) - 1;
    constexpr int kPer = 32 / BITS;
    __shared__ uint32_t scratch[kWarpsPerCta][8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwords = p.nnz / kPer;
    const long long rows = static_cast<long long>(p.units) * p.tokens;
    for (long long row = static_cast<long long>(blockIdx.x) * kWarpsPerCta + warp; row < rows;
         row += static_cast<long long>(gridDim.x) * kWarpsPerCta) {
        const int unit = static_cast<int>(row / p.tokens), t = static_cast<int>(row % p.tokens);
        const Residual res = load_residual(p, unit, t, lane);
        bool keep[4];
        uint32_t vote[4];
        select_topk(res.key, p.nnz, lane, keep, vote);
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) amax = fmaxf(amax, keep[i] ? fabsf(res.r[i]) : 0.f);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, off));
        const __half hs = quant_scale<kQmax>(amax);
        const float s = __half2float(hs);
        if (lane < 8) scratch[warp][lane] = 0u;
        __syncwarp();
        const uint32_t below = (1u << lane) - 1u;
        int base = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (keep[i]) {
                const int q = quant_code<kQmax>(res.r[i], s);
                const int r = base + __popc(vote[i] & below);
                atomicOr(&scratch[warp][r / kPer], (static_cast<uint32_t>(q) & ((1u << BITS) - 1u)) << ((r % kPer) * BITS));
            }
            base += __popc(vote[i]);
        }
        __syncwarp();
        const size_t orow = static_cast<size_t>(unit) * p.out_stride + t;
        if (lane < nwords) static_cast<int32_t*>(p.payload)[orow * nwords + lane] = static_cast<int32_t>(scratch[warp][lane]);
        if (lane == 0) {
            uint4 bm;  // word w of the bitmap: coordinate d at bit 63 - d % 64
            bm.y = __brev(vote[0]);
            bm.x = __brev(vote[1]);
            bm.w = __brev(vote[2]);
            bm.z = __brev(vote[3]);
            static_cast<uint4*>(p.meta)[orow] = bm;
            p.scale[orow] = hs;
        }
        __syncwarp();
    }
}

int check_common(const char* who, const void* x, const void* cen, const void* ids, const void* payload, int batch,
                 int kv_heads, int tokens, int64_t x_stride, int clusters, int64_t out_stride) {
    if (!x || !cen || !ids || !payload) return fail(RESKV_ERR_INVALID, "%s: null tensor pointer", who);
    if (batch < 1 || kv_heads < 1 || tokens < 1) return fail(RESKV_ERR_INVALID, "%s: batch, heads and tokens must be positive", who);
    if (clusters < 1 || clusters > kMaxClusters) return fail(RESKV_ERR_INVALID, "%s: centroid count must be in [1,64]", who);
    if (x_stride < tokens || out_stride < tokens) return fail(RESKV_ERR_INVALID, "%s: token stride smaller than token count", who);
    if (int rc = check_device_pointer(x, who, "x")) return rc;
    return check_device_pointer(payload, who, "payload");
}

int grid_for(long long rows) {
    const long long want = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
    const long long cap = static_cast<long long>(sm_count()) * 16;
    return static_cast<int>(want < cap ? want : cap);
}

}  // namespace
}  // namespace reskv

using namespace reskv;

extern "C" int reskv_encode_bitmap_fp16(const void* x, const void* centroids, const int32_t* ids, int batch,
                                        int kv_heads, int tokens, int64_t x_tok_stride, int clusters, int nnz,
                                        void* payload, void* bitmap, int64_t out_tok_stride, void* stream) {
    if (int rc = check_common("encode_bitmap_fp16", x, centroids, ids, payload, batch, kv_heads, tokens, x_tok_stride,
                              clusters, out_tok_stride))
        return rc;
    if (!bitmap || !aligned16(bitmap)) return fail(RESKV_ERR_INVALID, "encode_bitmap_fp16: bitmap must be a 16-byte aligned pointer");
    if (nnz < 1 || nnz > 127) return fail(RESKV_ERR_INVALID, "encode_bitmap_fp16: nnz must be in [1,127], got %d", nnz);
    EncodeParams p{static_cast<const __half*>(x), static_cast<const __half*>(centroids), ids, payload, bitmap, nullptr,
                   x_tok_stride, out_tok_stride, batch * kv_heads, tokens, clusters, nnz};
    if (!aligned16(x) || !aligned16(centroids) || !aligned16(payload))
        return fail(RESKV_ERR_INVALID, "encode_bitmap_fp16: x, centroids and payload must be 16-byte aligned");
    return launch_topk_bitmap_fp16(p, static_cast<cudaStream_t>(stream));
}

extern "C" int reskv_encode_quantized(const void* x, const void* centroids, const int32_t* ids, int batch, int kv_heads,
                                      int tokens, int64_t x_tok_stride, int clusters, int nnz, int bits, void* words,
                                      void* scale, int64_t out_tok_stride, void* stream) {
    if (int rc = check_common("encode_quantized", x, centroids, ids, words, batch, kv_heads, tokens, x_tok_stride,
                              clusters, out_tok_stride))
        return rc;
    if (!scale) return fail(RESKV_ERR_INVALID, "encode_quantized: null scale pointer");
    if (nnz != 32 && nnz != 64) return fail(RESKV_ERR_INVALID, "encode_quantized: nnz must be 32 or 64, got %d", nnz);
    if (bits != 2 && bits != 4) return fail(RESKV_ERR_INVALID, "encode_quantized: bits must be 2 or 4, got %d", bits);
    EncodeParams p{static_cast<const __half*>(x), static_cast<const __half*>(centroids), ids, words, nullptr,
                   static_cast<__half*>(scale), x_tok_stride, out_tok_stride, batch * kv_heads, tokens, clusters, nnz};
    if (!aligned16(x) || !aligned16(centroids) || !aligned16(words))
        return fail(RESKV_ERR_INVALID, "encode_quantized: x, centroids and words must be 16-byte aligned");
    return launch_topk_quantized(p, bits, static_cast<cudaStream_t>(stream));
}

extern "C" int reskv_encode_compact(const void* x, const void* centroids, const int32_t* ids, int batch, int kv_heads,
                                    int tokens, int64_t x_tok_stride, int clusters, int nnz, int bits, void* words,
                                    void* bitmap, void* scale, int64_t out_tok_stride, void* stream) {
    if (int rc = check_common("encode_compact", x, centroids, ids, words, batch, kv_heads, tokens, x_tok_stride,
                              clusters, out_tok_stride))
        return rc;
    if (!scale || !bitmap) return fail(RESKV_ERR_INVALID, "encode_compact: null bitmap or scale pointer");
    if (nnz != 32 && nnz != 64) return fail(RESKV_ERR_INVALID, "encode_compact: nnz must be 32 or 64, got %d", nnz);
    if (bits != 2 && bits != 4) return fail(RESKV_ERR_INVALID, "encode_compact: bits must be 2 or 4, got %d", bits);
    if (nnz * bits < 128) return fail(RESKV_ERR_INVALID, "encode_compact: rows below 16 bytes (nnz %d, %d bits) are not supported", nnz, bits);
    EncodeParams p{static_cast<const __half*>(x), static_cast<const __half*>(centroids), ids, words, bitmap,
                   static_cast<__half*>(scale), x_tok_stride, out_tok_stride, batch * kv_heads, tokens, clusters, nnz};
    const long long rows = static_cast<long long>(p.units) * tokens;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (bits == 4)
        encode_compact_kernel<4><<<grid_for(rows), kWarpsPerCta * 32, 0, s>>>(p);
    else
        encode_compact_kernel<2><<<grid_for(rows), kWarpsPerCta * 32, 0, s>>>(p);
    return check_cuda(cudaGetLastError(), "encode_compact launch");
}

extern "C" int reskv_encode_tiled_fp16(const void* x, const void* centroids, const int32_t* ids, int batch,
                                       int kv_heads, int tokens, int64_t x_tok_stride, int clusters, int nnz,
                                       int structured, void* values, void* meta, int64_t out_tok_stride, void* stream) {
    if (int rc = check_common("encode_tiled_fp16", x, centroids, ids, values, batch, kv_heads, tokens, x_tok_stride,
                              clusters, out_tok_stride))
        return rc;
    if (!meta) return fail(RESKV_ERR_INVALID, "encode_tiled_fp16: null metadata pointer");
    if (nnz <= 0 || nnz >= 128 || nnz % 8) return fail(RESKV_ERR_INVALID, "encode_tiled_fp16: nnz must be a multiple of 8 below 128, got %d", nnz);
    if (structured && nnz != 32) return fail(RESKV_ERR_INVALID, "encode_tiled_fp16: the 4:16 index form needs nnz == 32");
    EncodeParams p{static_cast<const __half*>(x), static_cast<const __half*>(centroids), ids, values, meta, nullptr,
                   x_tok_stride, out_tok_stride, batch * kv_heads, tokens, clusters, nnz};
    if (!aligned16(x) || !aligned16(centroids) || !aligned16(values) || !aligned16(meta))
        return fail(RESKV_ERR_INVALID, "encode_tiled_fp16: x, centroids, values and meta must be 16-byte aligned");
    return launch_topk_tiled_fp16(p, structured != 0, static_cast<cudaStream_t>(stream));
}

extern "C" int reskv_encode_structured_int4(const void* x, const void* centroids, const int32_t* ids, int batch,
                                            int kv_heads, int tokens, int64_t x_tok_stride, int clusters, void* packed,
                                            void* meta, void* scale, int64_t out_tok_stride, void* stream) {
    if (int rc = check_common("encode_structured_int4", x, centroids, ids, packed, batch, kv_heads, tokens,
                              x_tok_stride, clusters, out_tok_stride))
        return rc;
    if (!meta || !scale) return fail(RESKV_ERR_INVALID, "encode_structured_int4: null metadata or scale pointer");
    EncodeParams p{static_cast<const __half*>(x), static_cast<const __half*>(centroids), ids, packed, meta,
                   static_cast<__half*>(scale), x_tok_stride, out_tok_stride, batch * kv_heads, tokens, clusters, 32};
    if (!aligned16(x) || !aligned16(centroids) || !aligned16(packed) || (reinterpret_cast<uintptr_t>(meta) & 7u) != 0)
        return fail(RESKV_ERR_INVALID, "encode_structured_int4: x, centroids and packed must be 16-byte, meta 8-byte aligned");
    return launch_topk_structured_int4(p, static_cast<cudaStream_t>(stream));
}

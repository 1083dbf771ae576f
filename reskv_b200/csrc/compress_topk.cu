// Residual packers of the two layouts that keep the globally largest residuals of a token
// (unstructured FP16 bitmap; unstructured INT4 / INT2): one THREAD per token.
//
// The warp-per-token form spends most of its instructions on cross-lane traffic: every round of the
// threshold bisection ends in a warp reduction, ranks and masks are votes and popcounts.  With a whole
// token in one thread nothing crosses lanes:
//
//   * a warp stages the rows of 32 consecutive tokens in shared memory with 16-byte asynchronous copies
//     (rows 16 bytes apart from dense, so the 16-byte loads of eight lanes fall into distinct banks), the
//     unit's centroid table is staged once per CTA;
//   * the thread forms r = fp32(x) - fp32(c) and keeps the 128 selection keys |fp16(r)| as 64 packed pairs;
//     the pairing is (coordinate a + 16 in the low half, coordinate a in the high half), which makes the
//     masks of the packed comparisons fall straight onto the MSB-first bitmap words;
//   * the k-th largest key is found by bisection on its 15 bits: a round is 64 packed comparisons (1.0 / 0.0
//     per half, integer pipe) summed by packed FP16 additions (floating-point pipe), two instructions per key
//     pair and round on two different pipes;
//   * ties at the threshold keep the lower coordinates; the kept FP16 residuals are compacted in place in
//     the thread's own row and the warp writes the 32 rows out with 16-byte stores.
//
// Rounding points are those of compress.cu (they decide bit-exactness): selection key |fp16(r)|, FP16 layouts
// store fp16(r), the quantisers divide the FP32 r with the approximate division of the reference's build.
#include <cuda_fp16.h>

#include "compress_common.cuh"

namespace reskv {
namespace {

constexpr int kTopkWarps = 4;                 // warps per CTA
constexpr int kTopkThreads = kTopkWarps * 32;
constexpr int kRowBytes = 2 * kHeadDim + 16;  // shared-memory row of one token / one centroid
constexpr int kChunkTokens = kTopkThreads;    // tokens a CTA takes per pass (32 per warp)

enum class TopkMode { kBitmapFp16, kQuant4, kQuant2 };

__device__ __forceinline__ float half_lo(uint32_t v) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(v & 0xffffu)));
}
__device__ __forceinline__ float half_hi(uint32_t v) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(v >> 16)));
}
__device__ __forceinline__ __half2 as_half2(uint32_t v) { return *reinterpret_cast<const __half2*>(&v); }
__device__ __forceinline__ uint32_t as_u32(__half2 v) { return *reinterpret_cast<const uint32_t*>(&v); }

// r[q] = fp32(x[32 p + q]) - fp32(c[32 p + q]), q = 0..31, from the token's and its centroid's shared-memory rows
__device__ __forceinline__ void residual_piece(const unsigned char* xrow, const unsigned char* crow, int p,
                                               float (&r)[32]) {
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xrow + 64 * p + 16 * m);
        const uint4 cv = *reinterpret_cast<const uint4*>(crow + 64 * p + 16 * m);
        const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, cs[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            r[8 * m + 2 * i] = half_lo(xs[i]) - half_lo(cs[i]);
            r[8 * m + 2 * i + 1] = half_hi(xs[i]) - half_hi(cs[i]);
        }
    }
}

// Keep-mask of the `k` largest keys, lower coordinate first among equal keys.  key[16 p + j] holds coordinate
// 32 p + 16 + j in its low and 32 p + j in its high half; keep[p] has coordinate 32 p + q at bit 31 - q.
__device__ __forceinline__ void select_topk_thread(const uint32_t (&key)[64], int k, uint32_t (&keep)[4]) {
    // largest v with count(key >= v) >= k
    uint32_t v = 0;
    int n_ge = kHeadDim;
    for (int bit = 14; bit >= 0; --bit) {
        const uint32_t cand = v | (1u << bit);
        const __half2 c2 = as_half2(cand | (cand << 16));
        // the comparisons (1.0 / 0.0 per half) issue on the integer pipe, their sums on the FP16 pipe; counts up
        // to 128 are exact in FP16; four accumulators keep the addition chains short
        __half2 acc[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[u] = __hge2(as_half2(key[u]), c2);
#pragma unroll
        for (int j = 4; j < 64; ++j) acc[j & 3] = __hadd2(acc[j & 3], __hge2(as_half2(key[j]), c2));
        const __half2 total = __hadd2(__hadd2(acc[0], acc[1]), __hadd2(acc[2], acc[3]));
        const int cnt = __half2int_rn(__hadd(__low2half(total), __high2half(total)));
        if (cnt >= k) v = cand, n_ge = cnt;
    }
    const __half2 v2 = as_half2(v | (v << 16));
    uint32_t ge[4] = {0u, 0u, 0u, 0u}, gt[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int p = 0; p < 4; ++p) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t place = (0x80000000u >> j) | (0x8000u >> j);
            ge[p] |= __hge2_mask(as_half2(key[16 * p + j]), v2) & place;
            gt[p] |= __hgt2_mask(as_half2(key[16 * p + j]), v2) & place;
        }
    }
    if (n_ge == k) {
#pragma unroll
        for (int p = 0; p < 4; ++p) keep[p] = ge[p];
        return;
    }
    // more keys equal to the threshold than places left: the lowest coordinates among them stay
    int need = k - (__popc(gt[0]) + __popc(gt[1]) + __popc(gt[2]) + __popc(gt[3]));
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        uint32_t eq = ge[p] ^ gt[p], kept = gt[p];
        while (eq != 0u && need > 0) {
            const uint32_t first = 0x80000000u >> __clz(eq);
            eq ^= first, kept |= first, --need;
        }
        keep[p] = kept;
    }
}

template <TopkMode MODE>
__global__ void __launch_bounds__(kTopkThreads, 4) encode_topk_kernel(const EncodeParams p) {
    extern __shared__ __align__(16) unsigned char topk_smem[];
    unsigned char* cen_s = topk_smem;                                                 // [clusters][kRowBytes]
    unsigned char* rows_s = topk_smem + static_cast<size_t>(p.clusters) * kRowBytes;  // [warps][32][kRowBytes]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned char* my_rows = rows_s + static_cast<size_t>(warp) * 32 * kRowBytes;
    unsigned char* xrow = my_rows + lane * kRowBytes;
    const int chunks_per_unit = (p.tokens + kChunkTokens - 1) / kChunkTokens;
    const long long chunks = static_cast<long long>(p.units) * chunks_per_unit;
    int staged_unit = -1;
    for (long long c = blockIdx.x; c < chunks; c += gridDim.x) {
        const int unit = static_cast<int>(c / chunks_per_unit);
        const int t0 = static_cast<int>(c % chunks_per_unit) * kChunkTokens + warp * 32;
        const int ntok = max(0, min(32, p.tokens - t0));
        if (unit != staged_unit) {  // uniform over the CTA
            __syncthreads();        // nobody still reads the previous table
            const unsigned char* src = reinterpret_cast<const unsigned char*>(p.cen + static_cast<size_t>(unit) * p.clusters * kHeadDim);
            for (int i = tid; i < p.clusters * 16; i += kTopkThreads) cp_async16(cen_s + (i >> 4) * kRowBytes + (i & 15) * 16, src + i * 16);
            staged_unit = unit;
        }
        {
            const unsigned char* src = reinterpret_cast<const unsigned char*>(p.x + (static_cast<size_t>(unit) * p.x_stride + t0) * kHeadDim);
            for (int i = lane; i < ntok * 16; i += 32) cp_async16(my_rows + (i >> 4) * kRowBytes + (i & 15) * 16, src + i * 16);
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();  // table and rows in place (uniform: every thread of the CTA gets here every pass)

        uint32_t keep[4] = {0u, 0u, 0u, 0u};
        const size_t orow = static_cast<size_t>(unit) * p.out_stride + t0 + lane;
        if (lane < ntok) {
            int id = p.ids[static_cast<size_t>(unit) * p.tokens + t0 + lane];
            id = min(max(id, 0), p.clusters - 1);
            const unsigned char* crow = cen_s + id * kRowBytes;
            uint32_t key[64];
#pragma unroll
            for (int pc = 0; pc < 4; ++pc) {
                float r[32];
                residual_piece(xrow, crow, pc, r);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    key[16 * pc + j] = as_u32(__floats2half2_rn(r[16 + j], r[j])) & 0x7fff7fffu;
                if constexpr (MODE == TopkMode::kBitmapFp16) {
                    // fp16(r) in coordinate order replaces the (fully consumed) x values of this piece
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        uint4 o;
                        o.x = as_u32(__floats2half2_rn(r[8 * m], r[8 * m + 1]));
                        o.y = as_u32(__floats2half2_rn(r[8 * m + 2], r[8 * m + 3]));
                        o.z = as_u32(__floats2half2_rn(r[8 * m + 4], r[8 * m + 5]));
                        o.w = as_u32(__floats2half2_rn(r[8 * m + 6], r[8 * m + 7]));
                        *reinterpret_cast<uint4*>(xrow + 64 * pc + 16 * m) = o;
                    }
                }
            }
            select_topk_thread(key, p.nnz, keep);

            if constexpr (MODE == TopkMode::kBitmapFp16) {
                // compact the kept values to the front of the row (write index <= read index throughout)
                unsigned short* vals = reinterpret_cast<unsigned short*>(xrow);
                int n = 0;
#pragma unroll
                for (int pc = 0; pc < 4; ++pc) {
                    uint32_t w = keep[pc];
                    while (w != 0u) {
                        const int q = __clz(w);
                        w ^= 0x80000000u >> q;
                        vals[n++] = vals[32 * pc + q];
                    }
                }
                // bitmap words: coordinate d at bit 63 - d % 64 of word d / 64
                static_cast<uint4*>(p.meta)[orow] = make_uint4(keep[1], keep[0], keep[3], keep[2]);
            } else {
                constexpr int kBits = MODE == TopkMode::kQuant4 ? 4 : 2;
                constexpr int kQmax = (1 << (kBits - 1)) - 1;
                constexpr int kPer = 32 / kBits;  // codes per word
                // Two more passes over the residuals (largest kept magnitude, then the codes); the pieces are
                // taken one at a time (no unrolling over pc) so that only 32 residuals are live at once.
                float amax = 0.f;
#pragma unroll 1
                for (int pc = 0; pc < 4; ++pc) {
                    const uint32_t kw = pc == 0 ? keep[0] : pc == 1 ? keep[1] : pc == 2 ? keep[2] : keep[3];
                    float r[32];
                    residual_piece(xrow, crow, pc, r);
#pragma unroll
                    for (int q = 0; q < 32; ++q)
                        if (kw & (0x80000000u >> q)) amax = fmaxf(amax, fabsf(r[q]));
                }
                const __half hs = quant_scale<kQmax>(amax);
                const float s = __half2float(hs);
                uint32_t* words = reinterpret_cast<uint32_t*>(p.payload) + orow * (4 * kBits);
#pragma unroll 1
                for (int pc = 0; pc < 4; ++pc) {
                    const uint32_t kw = pc == 0 ? keep[0] : pc == 1 ? keep[1] : pc == 2 ? keep[2] : keep[3];
                    float r[32];
                    residual_piece(xrow, crow, pc, r);
                    uint32_t out[32 / kPer];
#pragma unroll
                    for (int w = 0; w < 32 / kPer; ++w) {
                        uint32_t word = 0u;
#pragma unroll
                        for (int i = 0; i < kPer; ++i) {
                            const int q = w * kPer + i;
                            if (kw & (0x80000000u >> q))
                                word |= (static_cast<uint32_t>(quant_code<kQmax>(r[q], s)) & ((1u << kBits) - 1u)) << (i * kBits);
                        }
                        out[w] = word;
                    }
                    // coordinates 32 pc .. 32 pc + 31 = words (32 / kPer) pc ...
                    if constexpr (kBits == 4) {
                        *reinterpret_cast<uint4*>(words + 4 * pc) = make_uint4(out[0], out[1], out[2], out[3]);
                    } else {
                        *reinterpret_cast<uint2*>(words + 2 * pc) = make_uint2(out[0], out[1]);
                    }
                }
                p.scale[orow] = hs;
            }
        }
        if constexpr (MODE == TopkMode::kBitmapFp16) {
            __syncwarp();
            // the warp's rows are consecutive in the output: 16-byte pieces when the row length allows it
            unsigned char* dst = reinterpret_cast<unsigned char*>(static_cast<__half*>(p.payload) +
                                                                  (static_cast<size_t>(unit) * p.out_stride + t0) * p.nnz);
            if (p.nnz % 8 == 0) {
                const int pieces = p.nnz / 8;
                for (int i = lane; i < ntok * pieces; i += 32) {
                    const int row = i / pieces, piece = i % pieces;
                    *reinterpret_cast<uint4*>(dst + static_cast<size_t>(row) * p.nnz * 2 + piece * 16) =
                        *reinterpret_cast<const uint4*>(my_rows + row * kRowBytes + piece * 16);
                }
            } else {
                for (int i = lane; i < ntok * p.nnz; i += 32) {
                    const int row = i / p.nnz, e = i % p.nnz;
                    reinterpret_cast<unsigned short*>(dst)[i] =
                        *reinterpret_cast<const unsigned short*>(my_rows + row * kRowBytes + e * 2);
                }
            }
        }
        __syncthreads();  // rows are rewritten by the next pass
    }
}

size_t topk_smem_bytes(int clusters) {
    return static_cast<size_t>(clusters + kTopkWarps * 32) * kRowBytes;
}

template <TopkMode MODE>
int launch_topk(const EncodeParams& p, cudaStream_t stream, const char* what) {
    auto kern = encode_topk_kernel<MODE>;
    // the kernel's shared memory grows with the centroid count: allow the maximum once per device
    static unsigned long long allowed = 0;
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    if (dev < 0 || dev >= 64 || !(allowed >> dev & 1ull)) {
        if (int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     static_cast<int>(topk_smem_bytes(kMaxClusters))), what))
            return rc;
        if (dev >= 0 && dev < 64) allowed |= 1ull << dev;
    }
    const long long chunks = static_cast<long long>(p.units) * ((p.tokens + kChunkTokens - 1) / kChunkTokens);
    const long long cap = static_cast<long long>(sm_count()) * 4;
    const int grid = static_cast<int>(chunks < cap ? chunks : cap);
    kern<<<grid, kTopkThreads, topk_smem_bytes(p.clusters), stream>>>(p);
    return check_cuda(cudaGetLastError(), what);
}

}  // namespace

int launch_topk_bitmap_fp16(const EncodeParams& p, cudaStream_t stream) {
    return launch_topk<TopkMode::kBitmapFp16>(p, stream, "encode_bitmap_fp16 launch");
}

int launch_topk_quantized(const EncodeParams& p, int bits, cudaStream_t stream) {
    return bits == 4 ? launch_topk<TopkMode::kQuant4>(p, stream, "encode_quantized launch")
                     : launch_topk<TopkMode::kQuant2>(p, stream, "encode_quantized launch");
}

}  // namespace reskv

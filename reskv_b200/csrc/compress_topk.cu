// Residual packers, one THREAD per token: the layouts that keep the globally largest residuals of a token
// (unstructured FP16 bitmap; unstructured INT4 / INT2), the layouts that keep the largest of every 16-coordinate
// tile (tiled masks, 4:16 indices) and the 1-of-4 INT4 layout.
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
// The tiled layouts run the same bisection per tile, two tiles at a time in the two halves of the packed
// operations (the accept decision is a packed comparison as well, so nothing is ever unpacked); the 1-of-4 layout
// compares four keys per group.
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

enum class TopkMode { kBitmapFp16, kQuant4, kQuant2, kTiledFp16, kStructFp16, kStructInt4 };

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

// Keep-mask of the `m` largest keys of every 16-coordinate tile, lower coordinate first among equal keys.
// key[16 p + j] holds coordinate 32 p + j (tile 2 p) in its LOW and 32 p + 16 + j (tile 2 p + 1) in its HIGH half;
// keep[p] has coordinate 32 p + q at bit q (the tiled metadata word of the reference, compression.cu:126-139).
__device__ __forceinline__ void select_tiles_thread(const uint32_t (&key)[64], int m, uint32_t (&keep)[4]) {
    const __half2 m2 = __float2half2_rn(static_cast<float>(m));
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        // per half: largest v with count(key >= v) >= m; counts up to 16 are exact in FP16
        uint32_t v2 = 0;
        for (int bit = 14; bit >= 0; --bit) {
            const uint32_t both = (1u << bit) | (1u << (bit + 16));
            const __half2 c2 = as_half2(v2 | both);
            __half2 a0 = __hge2(as_half2(key[16 * p]), c2), a1 = __hge2(as_half2(key[16 * p + 1]), c2);
#pragma unroll
            for (int j = 2; j < 16; j += 2) {
                a0 = __hadd2(a0, __hge2(as_half2(key[16 * p + j]), c2));
                a1 = __hadd2(a1, __hge2(as_half2(key[16 * p + j + 1]), c2));
            }
            v2 |= both & __hge2_mask(__hadd2(a0, a1), m2);  // each half accepts the bit on its own count
        }
        const __half2 t2 = as_half2(v2);
        uint32_t ge = 0u, gt = 0u;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t place = (1u << j) | (0x10000u << j);
            ge |= __hge2_mask(as_half2(key[16 * p + j]), t2) & place;
            gt |= __hgt2_mask(as_half2(key[16 * p + j]), t2) & place;
        }
        uint32_t kept = 0u;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t g = (ge >> (16 * h)) & 0xffffu, t = (gt >> (16 * h)) & 0xffffu;
            uint32_t k = g;
            if (__popc(g) != m) {  // more keys equal to the threshold than places left: the lowest coordinates stay
                int need = m - __popc(t);
                uint32_t eq = g ^ t;
                k = t;
                while (eq != 0u && need > 0) {
                    const uint32_t first = eq & (0u - eq);
                    eq ^= first, k |= first, --need;
                }
            }
            kept |= k << (16 * h);
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
        constexpr bool kTiles = MODE == TopkMode::kTiledFp16 || MODE == TopkMode::kStructFp16;
        constexpr bool kFp16Rows = MODE == TopkMode::kBitmapFp16 || kTiles;  // the row becomes the FP16 payload
        if constexpr (MODE == TopkMode::kStructInt4) {
            // one residual of every four consecutive coordinates: the largest |fp16(r)|, lowest index on ties;
            // FP32 scale amax / 7, codes with the approximate division (compression.cu:153-239)
            if (lane < ntok) {
                int id = p.ids[static_cast<size_t>(unit) * p.tokens + t0 + lane];
                id = min(max(id, 0), p.clusters - 1);
                const unsigned char* crow = cen_s + id * kRowBytes;
                uint32_t which[2] = {0u, 0u};  // 2-bit in-group index of group g at bit 2 (g % 16) of word g / 16
                float amax = 0.f;
#pragma unroll 1
                for (int pc = 0; pc < 4; ++pc) {
                    float r[32];
                    residual_piece(xrow, crow, pc, r);
                    uint32_t w = 0u;
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        uint32_t bk = __half_as_ushort(__float2half_rn(r[4 * g])) & 0x7fffu, bi = 0u;
                        float br = r[4 * g];
#pragma unroll
                        for (int e = 1; e < 4; ++e) {
                            const uint32_t k = __half_as_ushort(__float2half_rn(r[4 * g + e])) & 0x7fffu;
                            if (k > bk) bk = k, bi = e, br = r[4 * g + e];
                        }
                        amax = fmaxf(amax, fabsf(br));
                        w |= bi << (2 * g);
                    }
                    if (pc < 2) which[0] |= w << (16 * pc); else which[1] |= w << (16 * (pc - 2));
                }
                const float s = amax > 0.f ? amax * (1.0f / 7.0f) : 1.0f;
                uint32_t out[4];
#pragma unroll 1
                for (int pc = 0; pc < 4; ++pc) {
                    float r[32];
                    residual_piece(xrow, crow, pc, r);
                    const uint32_t w = (pc < 2 ? which[0] >> (16 * pc) : which[1] >> (16 * (pc - 2))) & 0xffffu;
                    uint32_t word = 0u;
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        const uint32_t bi = (w >> (2 * g)) & 3u;
                        const float br = bi == 0u ? r[4 * g] : bi == 1u ? r[4 * g + 1] : bi == 2u ? r[4 * g + 2] : r[4 * g + 3];
                        const int q = max(-7, min(7, __float2int_rn(div_fast(br, s))));
                        word |= (static_cast<uint32_t>(q) & 15u) << (4 * g);
                    }
                    if (pc == 0) out[0] = word; else if (pc == 1) out[1] = word; else if (pc == 2) out[2] = word; else out[3] = word;
                }
                const size_t orow = static_cast<size_t>(unit) * p.out_stride + t0 + lane;
                static_cast<uint4*>(p.payload)[orow] = make_uint4(out[0], out[1], out[2], out[3]);
                static_cast<uint2*>(p.meta)[orow] = make_uint2(which[0], which[1]);
                p.scale[orow] = __float2half_rn(s);
            }
            __syncthreads();  // rows are rewritten by the next pass
            continue;
        }
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
                    key[16 * pc + j] = as_u32(kTiles ? __floats2half2_rn(r[j], r[16 + j]) : __floats2half2_rn(r[16 + j], r[j])) & 0x7fff7fffu;
                if constexpr (kFp16Rows) {
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
            if constexpr (kTiles) {
                select_tiles_thread(key, p.nnz / 8, keep);
                // compact the kept values to the front of the row, ascending coordinates (= tile, then rank)
                unsigned short* vals = reinterpret_cast<unsigned short*>(xrow);
                int n = 0;
                uint32_t code[4] = {0u, 0u, 0u, 0u};  // 4:16 form: four 4-bit in-tile indices per tile, rank r at bit 4 r
#pragma unroll
                for (int pc = 0; pc < 4; ++pc) {
                    uint32_t w = keep[pc];
                    int rank = 0;
                    while (w != 0u) {
                        const int q = __ffs(w) - 1;
                        w &= w - 1u;
                        vals[n++] = vals[32 * pc + q];
                        if constexpr (MODE == TopkMode::kStructFp16) {
                            // ranks restart at the second tile of the word (bit 16): four values per tile
                            code[pc] |= static_cast<uint32_t>(q & 15) << (4 * (rank & 3) + (q & 16));
                            ++rank;
                        }
                    }
                }
                if constexpr (MODE == TopkMode::kStructFp16)
                    static_cast<uint4*>(p.meta)[orow] = make_uint4(code[0], code[1], code[2], code[3]);
                else
                    static_cast<uint4*>(p.meta)[orow] = make_uint4(keep[0], keep[1], keep[2], keep[3]);
            } else {
                select_topk_thread(key, p.nnz, keep);
            }

            if constexpr (kTiles) {
            } else if constexpr (MODE == TopkMode::kBitmapFp16) {
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
        if constexpr (kFp16Rows) {
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

int launch_topk_tiled_fp16(const EncodeParams& p, bool indexed, cudaStream_t stream) {
    return indexed ? launch_topk<TopkMode::kStructFp16>(p, stream, "encode_tiled_fp16 launch")
                   : launch_topk<TopkMode::kTiledFp16>(p, stream, "encode_tiled_fp16 launch");
}

int launch_topk_structured_int4(const EncodeParams& p, cudaStream_t stream) {
    return launch_topk<TopkMode::kStructInt4>(p, stream, "encode_structured_int4 launch");
}

int launch_topk_quantized(const EncodeParams& p, int bits, cudaStream_t stream) {
    return bits == 4 ? launch_topk<TopkMode::kQuant4>(p, stream, "encode_quantized launch")
                     : launch_topk<TopkMode::kQuant2>(p, stream, "encode_quantized launch");
}

}  // namespace reskv

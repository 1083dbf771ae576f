// Lloyd clustering of pre-RoPE K or V per (sequence, KV head): fused assignment +
// centroid accumulation, centroid update, and the decode-time incremental step.
//
// Assignment is the exact nearest centre in FP32 (squared differences summed in
// a fixed order), lowest index on ties.  The bulk of it runs on the tensor cores:
// |c|^2 - 2 x.c for 16 tokens x 8 centres per mma.sync (centres split into FP16
// hi + lo so the products are exact), which ranks the centres up to an error far
// below the FP32 sum's own; a token whose two best candidates are closer than a
// conservative bound on that error is re-ranked by the exact FP32 sum, so the
// ids are those of the exact computation.  Cluster sums are accumulated *exactly*:
// an FP16 value is an integer multiple of 2^-24, so tokens are added as 2^24-
// scaled integers (split into two 32-bit shared-memory counters per CTA, flushed
// with 64-bit integer atomics).  Integer addition is associative, which makes
// the new centres independent of scheduling and equal to the correctly rounded
// mean -- results are reproducible run to run.
//
// That exact accumulation costs ~100 warp instructions per token (128 coordinates x two shared-memory atomics).
// The default for up to 32 centres is therefore a second form that keeps the exact *assignment* but forms the
// cluster sums on the tensor cores as onehot(ids)^T . X (the token rows are already in registers as MMA
// operands; movmatrix turns them into the other operand), FP32 accumulators per warp, warps added in index
// order, and the CTA's FP32 partial sums flushed as 2^24-scaled integers.  Every step has a fixed order or is
// an integer addition, so results are still reproducible run to run; the means can differ from the correctly
// rounded ones by FP32 rounding of the partial sums (checked: within one FP16 unit in the last place).
//
// K flavour: FP32 centres, an empty cluster keeps its centre.
// V flavour: centres rounded to FP16 after every update, an empty cluster becomes 0.
#include <cuda.h>  // CUtensorMap and its enums; the encoder itself is looked up at run time

#include "common.cuh"

namespace reskv {
namespace {

constexpr uint32_t kFull = 0xffffffffu;
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kChunk = 512;  // tokens per CTA, exact accumulation: keeps the split 32-bit counters from overflowing
constexpr int kChunkFastMax = 4096;  // most tokens per CTA with tensor-core accumulation
constexpr int kRedStride = 132;   // floats per cluster row of the cross-warp reduction buffer
constexpr int kXsRow = 2 * kHeadDim + 16;  // bytes per staged token row (16-byte loads of eight lanes in distinct banks)
constexpr float kFix = 16777216.0f;  // 2^24

struct KmeansParams {
    const __half* x;       // [units, x_stride, 128]
    float* centres;        // [units, C, 128] working centres (FP32 values)
    long long* sums;       // [units, C, 128] 2^24-scaled integer sums, zero on entry
    int* counts;           // [units, C], zero on entry
    int32_t* ids;          // [units, tokens]
    uint32_t* status;      // RESKV_STATUS_* bits (a bounded wait that ran out); cleared by the init kernel
    int64_t x_stride;
    int units, tokens, clusters;
};

struct InitIndex {
    int idx[kMaxClusters];
};

__global__ void kmeans_init_kernel(KmeansParams p, InitIndex init, int value) {
    const int unit = blockIdx.x;
    for (int i = threadIdx.x; i < p.clusters * kHeadDim; i += blockDim.x) {
        const int c = i / kHeadDim, d = i % kHeadDim;
        const float v = __half2float(p.x[(static_cast<size_t>(unit) * p.x_stride + init.idx[c]) * kHeadDim + d]);
        p.centres[(static_cast<size_t>(unit) * p.clusters + c) * kHeadDim + d] = v;
        p.sums[(static_cast<size_t>(unit) * p.clusters + c) * kHeadDim + d] = 0;
    }
    for (int c = threadIdx.x; c < p.clusters; c += blockDim.x) p.counts[unit * p.clusters + c] = 0;
    if (unit == 0 && threadIdx.x == 0) *p.status = 0u;
    (void)value;
}

// Squared distance of the warp's token to each centre, reduced so that lane c
// holds the total for centre cbase + c; returns (best distance, best index) in
// every lane.  `xv` are the lane's coordinates {lane + 32 i}.
__device__ __forceinline__ void nearest(const float* cen_s, int clusters, const float (&xv)[4], int lane, float& best,
                                        int& best_c) {
    best = INFINITY, best_c = 0;
    for (int cbase = 0; cbase < clusters; cbase += 32) {
        float part[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            float acc = 0.f;
            if (cbase + c < clusters) {
                const float* row = cen_s + (cbase + c) * kHeadDim;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float df = xv[i] - row[lane + 32 * i];
                    acc = fmaf(df, df, acc);
                }
            }
            part[c] = acc;
        }
        // transposing butterfly: after the step with offset `off`, a lane keeps the
        // half of its values whose centre index has the same `off` bit as the lane
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const bool up = lane & off;
#pragma unroll
            for (int c = 0; c < off; ++c) {
                const float send = up ? part[c] : part[c + off];
                const float keep = up ? part[c + off] : part[c];
                part[c] = keep + __shfl_xor_sync(kFull, send, off);
            }
        }
        float dist = (cbase + lane < clusters) ? part[0] : INFINITY;
        int idx = cbase + lane;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float od = __shfl_xor_sync(kFull, dist, off);
            const int oi = __shfl_xor_sync(kFull, idx, off);
            if (od < dist || (od == dist && oi < idx)) dist = od, idx = oi;
        }
        if (dist < best) best = dist, best_c = idx;  // earlier block wins ties
    }
}

constexpr int kCenHalfStride = 132;  // FP16 centre rows: stride = 2 banks mod 32, so B-fragment loads do not collide
constexpr float kTieBound = 1.0f / 32768.0f;  // re-rank when (d2 - d1) <= kTieBound * (|x|^2 + max |c|^2)

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Offset (in coordinates) of MMA k-step `ks` for quad lane `q`: a lane owns coordinates
// [16 q, 16 q + 16) and [64 + 16 q, 64 + 16 q + 16), four per k-step.
__device__ __forceinline__ int kstep_offset(int ks, int q) { return (ks < 4 ? 0 : 48) + 16 * q + 4 * ks; }

// grid (chunks, units).  Tensor-core assignment of the chunk's tokens (see the file header), then
// exact accumulation of sums and counts.  HILO = centres are FP32 (key flavour): use hi + lo FP16.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// FAST: cluster sums on the tensor cores (needs padded <= 32), else exact integer accumulation.
template <bool HILO, bool FAST>
__global__ void __launch_bounds__(kThreads) kmeans_assign_mma_kernel(const KmeansParams p, int padded, int chunk) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* cen_s = reinterpret_cast<float*>(smem);                              // [C][128] FP32 centres (exact path)
    int* lo_s = reinterpret_cast<int*>(cen_s + p.clusters * kHeadDim);          // [C][128] low 20 bits
    int* hi_s = lo_s + p.clusters * kHeadDim;                                   // [C][128] the rest
    // FAST uses the counter arrays' place for its FP32 reduction slabs [warps][32][kRedStride] (sized by the host)
    const int counter_ints = FAST ? kWarps * 32 * kRedStride : 2 * p.clusters * kHeadDim;
    int* cnt_s = lo_s + counter_ints;                                           // [C]
    float* cn_s = reinterpret_cast<float*>(cnt_s + kMaxClusters);               // [padded] |c|^2, +inf for padding
    __half* ch_s = reinterpret_cast<__half*>(cn_s + kMaxClusters);              // [padded][132] FP16 hi
    __half* cl_s = ch_s + padded * kCenHalfStride;                              // [padded][132] FP16 lo (HILO)
    __shared__ float cmax_s;
    const int unit = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q = lane & 3;
    const int t_begin = blockIdx.x * chunk, t_end = min(p.tokens, t_begin + chunk);
    const float* cen_g = p.centres + static_cast<size_t>(unit) * p.clusters * kHeadDim;
    for (int i = tid; i < p.clusters * kHeadDim; i += kThreads) {
        cen_s[i] = cen_g[i];
        lo_s[i] = 0;
        hi_s[i] = 0;
    }
    for (int i = tid; i < padded * kHeadDim; i += kThreads) {
        const int c = i / kHeadDim, d = i % kHeadDim;
        const float v = c < p.clusters ? cen_g[i] : 0.f;
        const __half h = __float2half_rn(v);
        ch_s[c * kCenHalfStride + d] = h;
        if (HILO) cl_s[c * kCenHalfStride + d] = __float2half_rn(v - __half2float(h));
    }
    for (int c = tid; c < kMaxClusters; c += kThreads) cnt_s[c] = 0;
    __syncthreads();
    // |c|^2 of the value the MMA actually sees (hi + lo), one warp per centre
    for (int c = warp; c < padded; c += kWarps) {
        float acc = 0.f;
        if (c < p.clusters) {
            for (int d = lane; d < kHeadDim; d += 32) {
                float v = __half2float(ch_s[c * kCenHalfStride + d]);
                if (HILO) v += __half2float(cl_s[c * kCenHalfStride + d]);
                acc = fmaf(v, v, acc);
            }
            for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(kFull, acc, off);
        } else {
            acc = INFINITY;
        }
        if (lane == 0) cn_s[c] = acc;
    }
    __syncthreads();
    if (tid == 0) {
        float m = 0.f;
        for (int c = 0; c < p.clusters; ++c) m = fmaxf(m, cn_s[c]);
        cmax_s = m;
    }
    __syncthreads();
    const float cmax = cmax_s;
    const __half* xu = p.x + static_cast<size_t>(unit) * p.x_stride * kHeadDim;
    // FAST: sums[cluster 16 mb + g (+8)][coordinate kstep_offset(ks, q) + 2 h + (0, 1)] of this warp's tokens,
    // n-block nb = 2 ks + h
    float acc_s[FAST ? 2 : 1][FAST ? 16 : 1][4];
    if constexpr (FAST) {
#pragma unroll
        for (int mb = 0; mb < 2; ++mb)
#pragma unroll
            for (int nb = 0; nb < 16; ++nb) acc_s[mb][nb][0] = acc_s[mb][nb][1] = acc_s[mb][nb][2] = acc_s[mb][nb][3] = 0.f;
    }

    // FAST: the warp's next 16 token rows travel to shared memory (16-byte asynchronous copies, rows 16 bytes
    // apart from dense) while the current block is being processed; the block is read into registers at the
    // top of the loop, which frees the buffer for the copy of the one after
    unsigned char* xs_w = reinterpret_cast<unsigned char*>(cl_s + (HILO ? padded * kCenHalfStride : 0)) + warp * 16 * kXsRow;
    auto stage_rows = [&](int t0) {
        const int n = min(16, t_end - t0);
        const unsigned char* src = reinterpret_cast<const unsigned char*>(xu + static_cast<size_t>(t0) * kHeadDim);
        for (int i = lane; i < n * 16; i += 32) cp_async16(xs_w + (i >> 4) * kXsRow + (i & 15) * 16, src + i * 16);
    };
    if constexpr (FAST) {
        if (t_begin + warp * 16 < t_end) stage_rows(t_begin + warp * 16);
    }

    for (int t0 = t_begin + warp * 16; t0 < t_end; t0 += kWarps * 16) {
        // A fragments: rows t0 + g and t0 + g + 8, the lane's 32 coordinates of each
        const int r0 = t0 + g, r1 = t0 + g + 8;
        uint32_t a[8][4];
        {
            uint4 v[2][4];
            if constexpr (FAST) {
                asm volatile("cp.async.wait_all;" ::: "memory");
                __syncwarp();
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int row = r ? r1 : r0;
                const uint4* src = FAST ? reinterpret_cast<const uint4*>(xs_w + (g + 8 * r) * kXsRow)
                                        : reinterpret_cast<const uint4*>(xu + static_cast<size_t>(row) * kHeadDim);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint4* at = src + (k < 2 ? 0 : 8) + 2 * q + (k & 1);
                    v[r][k] = row < t_end ? (FAST ? *at : __ldg(at)) : make_uint4(0, 0, 0, 0);
                }
            }
            if constexpr (FAST) {
                __syncwarp();  // every lane has its rows in registers
                if (t0 + kWarps * 16 < t_end) stage_rows(t0 + kWarps * 16);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                a[2 * k][0] = v[0][k].x, a[2 * k][1] = v[1][k].x, a[2 * k][2] = v[0][k].y, a[2 * k][3] = v[1][k].y;
                a[2 * k + 1][0] = v[0][k].z, a[2 * k + 1][1] = v[1][k].z, a[2 * k + 1][2] = v[0][k].w, a[2 * k + 1][3] = v[1][k].w;
            }
        }
        // |x|^2 of the 16 rows: diagonal of X X^T (B fragments are the A registers themselves)
        float xn0, xn1;
        {
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                mma_f16(s0, a[ks][0], a[ks][1], a[ks][2], a[ks][3], a[ks][0], a[ks][2]);
                mma_f16(s1, a[ks][0], a[ks][1], a[ks][2], a[ks][3], a[ks][1], a[ks][3]);
            }
            // row g x token g sits in lane (g, g / 2), element g % 2; row g + 8 x token g + 8 likewise in s1[2..3]
            const float mine0 = (g & 1) ? s0[1] : s0[0], mine1 = (g & 1) ? s1[3] : s1[2];
            xn0 = __shfl_sync(kFull, mine0, 4 * g + (g >> 1));
            xn1 = __shfl_sync(kFull, mine1, 4 * g + (g >> 1));
        }
        float d1[2] = {INFINITY, INFINITY}, d2[2] = {INFINITY, INFINITY};
        int c1[2] = {0, 0};
        // four centre blocks at a time: their accumulation chains are independent, which keeps the tensor pipe fed
        // with few resident warps (blocks beyond the padded count repeat the last one and are ignored)
        constexpr int kChains = 4;
        for (int nb0 = 0; nb0 < padded / 8; nb0 += kChains) {
            float acc[kChains][4];
            const __half* hrow[kChains];
            const __half* lrow[kChains];
#pragma unroll
            for (int h = 0; h < kChains; ++h) {
                acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
                const int nb = min(nb0 + h, padded / 8 - 1);
                hrow[h] = ch_s + (nb * 8 + g) * kCenHalfStride;
                lrow[h] = cl_s + (nb * 8 + g) * kCenHalfStride;
            }
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
                for (int h = 0; h < kChains; ++h) {
                    const uint2 bh = *reinterpret_cast<const uint2*>(hrow[h] + kstep_offset(ks, q));
                    mma_f16(acc[h], a[ks][0], a[ks][1], a[ks][2], a[ks][3], bh.x, bh.y);
                }
                if (HILO) {
#pragma unroll
                    for (int h = 0; h < kChains; ++h) {
                        const uint2 bl = *reinterpret_cast<const uint2*>(lrow[h] + kstep_offset(ks, q));
                        mma_f16(acc[h], a[ks][0], a[ks][1], a[ks][2], a[ks][3], bl.x, bl.y);
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < kChains; ++h) {
                if (nb0 + h >= padded / 8) break;
                const int col = (nb0 + h) * 8 + 2 * q;
                const float n0 = cn_s[col], n1 = cn_s[col + 1];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1, c = col + (e & 1);
                    const float d = fmaf(-2.f, acc[h][e], (e & 1) ? n1 : n0);
                    if (d < d1[r]) {
                        d2[r] = d1[r], d1[r] = d, c1[r] = c;
                    } else if (d < d2[r]) {
                        d2[r] = d;
                    }
                }
            }
        }
#pragma unroll
        for (int off = 1; off <= 2; off <<= 1) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float od1 = __shfl_xor_sync(kFull, d1[r], off), od2 = __shfl_xor_sync(kFull, d2[r], off);
                const int oc1 = __shfl_xor_sync(kFull, c1[r], off);
                if (od1 < d1[r] || (od1 == d1[r] && oc1 < c1[r])) {
                    d2[r] = fminf(d1[r], od2), d1[r] = od1, c1[r] = oc1;
                } else {
                    d2[r] = fminf(d2[r], od1);
                }
            }
        }
        // near-ties: re-rank with the exact FP32 sum (all lanes of the warp take part)
        const bool tie0 = r0 < t_end && (d2[0] - d1[0]) <= kTieBound * (xn0 + cmax);
        const bool tie1 = r1 < t_end && (d2[1] - d1[1]) <= kTieBound * (xn1 + cmax);
        uint32_t redo0 = __ballot_sync(kFull, tie0 && q == 0), redo1 = __ballot_sync(kFull, tie1 && q == 0);
        for (int half = 0; half < 2; ++half) {
            uint32_t redo = half ? redo1 : redo0;
            while (redo) {
                const int src = __ffs(redo) - 1;
                redo &= redo - 1;
                const int row = t0 + (src >> 2) + 8 * half;
                const __half* xr = xu + static_cast<size_t>(row) * kHeadDim;
                float xv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) xv[i] = __half2float(xr[lane + 32 * i]);
                float best;
                int c;
                nearest(cen_s, p.clusters, xv, lane, best, c);
                if ((lane >> 2) == (src >> 2)) c1[half] = c;
            }
        }
        if (q == 0) {
            if (r0 < t_end) p.ids[static_cast<size_t>(unit) * p.tokens + r0] = c1[0];
            if (r1 < t_end) p.ids[static_cast<size_t>(unit) * p.tokens + r1] = c1[1];
        }
        if constexpr (FAST) {
            // onehot(ids)^T . X: A = one-hot rows (cluster x token) from a packed FP16 compare of the ids, B = the
            // token rows transposed (movmatrix of the A fragments of the distance step); rows beyond the end are 0
            const int v0 = r0 < t_end ? c1[0] : -1, v1 = r1 < t_end ? c1[1] : -1;
            const int w0 = __shfl_sync(kFull, v0, 8 * q), w1 = __shfl_sync(kFull, v0, 8 * q + 4);
            const int w2 = __shfl_sync(kFull, v1, 8 * q), w3 = __shfl_sync(kFull, v1, 8 * q + 4);
            const __half2 gg = __half2half2(__int2half_rn(g));
            const __half2 d01 = __hsub2(__halves2half2(__int2half_rn(w0), __int2half_rn(w1)), gg);
            const __half2 d23 = __hsub2(__halves2half2(__int2half_rn(w2), __int2half_rn(w3)), gg);
            uint32_t oh[2][4];
#pragma unroll
            for (int mb = 0; mb < 2; ++mb) {
                const __half2 lo = __float2half2_rn(16.f * mb), hi = __float2half2_rn(16.f * mb + 8.f);
                const __half2 e0 = __heq2(d01, lo), e1 = __heq2(d01, hi), e2 = __heq2(d23, lo), e3 = __heq2(d23, hi);
                oh[mb][0] = *reinterpret_cast<const uint32_t*>(&e0), oh[mb][1] = *reinterpret_cast<const uint32_t*>(&e1);
                oh[mb][2] = *reinterpret_cast<const uint32_t*>(&e2), oh[mb][3] = *reinterpret_cast<const uint32_t*>(&e3);
            }
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t b00 = movmatrix_trans(a[ks][0]), b01 = movmatrix_trans(a[ks][1]);
                const uint32_t b10 = movmatrix_trans(a[ks][2]), b11 = movmatrix_trans(a[ks][3]);
#pragma unroll
                for (int mb = 0; mb < 2; ++mb) {
                    if (16 * mb < padded) {
                        mma_f16(acc_s[mb][2 * ks], oh[mb][0], oh[mb][1], oh[mb][2], oh[mb][3], b00, b01);
                        mma_f16(acc_s[mb][2 * ks + 1], oh[mb][0], oh[mb][1], oh[mb][2], oh[mb][3], b10, b11);
                    }
                }
            }
            if (q == 0) {
                if (r0 < t_end) atomicAdd(&cnt_s[c1[0]], 1);
                if (r1 < t_end) atomicAdd(&cnt_s[c1[1]], 1);
            }
            continue;
        }
        // exact accumulation, one token at a time with the warp across its coordinates
        const int rows = min(16, t_end - t0);
        for (int r = 0; r < rows; ++r) {
            const int c = __shfl_sync(kFull, (r & 8) ? c1[1] : c1[0], 4 * (r & 7));
            const __half* xr = xu + static_cast<size_t>(t0 + r) * kHeadDim;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // x * 2^24 is an integer below 2^41: split it, exactly, into hi * 2^20 + lo with both
                // parts carrying the sign of x (|lo| < 2^20, |hi| < 2^21)
                const float fx = __half2float(xr[lane + 32 * i]) * kFix;
                const float hi = truncf(fx * (1.0f / 1048576.0f));
                const float lo = fmaf(hi, -1048576.0f, fx);
                atomicAdd(&lo_s[c * kHeadDim + lane + 32 * i], __float2int_rz(lo));
                atomicAdd(&hi_s[c * kHeadDim + lane + 32 * i], __float2int_rz(hi));
            }
            if (lane == 0) atomicAdd(&cnt_s[c], 1);
        }
    }
    __syncthreads();
    long long* sums_g = p.sums + static_cast<size_t>(unit) * p.clusters * kHeadDim;
    if constexpr (FAST) {
        // every warp stores its partial sums in a slab of its own (the integer counters' memory, unused in this
        // form, enlarged by the host); the slabs are added in warp order and the CTA's sums go out as 2^24-scaled
        // integers
        float* red = reinterpret_cast<float*>(lo_s);  // [warps][32][kRedStride]
        {
            float* mine = red + warp * 32 * kRedStride;
#pragma unroll
            for (int mb = 0; mb < 2; ++mb)
#pragma unroll
                for (int nb = 0; nb < 16; ++nb)
#pragma unroll
                    for (int e = 0; e < 4; e += 2) {
                        const int cl = 16 * mb + g + 8 * (e >> 1);
                        const int d = kstep_offset(nb >> 1, q) + 2 * (nb & 1);
                        *reinterpret_cast<float2*>(mine + cl * kRedStride + d) = make_float2(acc_s[mb][nb][e], acc_s[mb][nb][e + 1]);
                    }
        }
        __syncthreads();
        for (int i = tid; i < p.clusters * kHeadDim; i += kThreads) {
            const int cl = i / kHeadDim, d = i % kHeadDim;
            if (cnt_s[cl] > 0) {
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) sum += red[(w * 32 + cl) * kRedStride + d];  // fixed order
                atomicAdd(reinterpret_cast<unsigned long long*>(sums_g + i),
                          static_cast<unsigned long long>(__float2ll_rn(sum * kFix)));
            }
        }
        for (int c = tid; c < p.clusters; c += kThreads)
            if (cnt_s[c] > 0) atomicAdd(&p.counts[unit * p.clusters + c], cnt_s[c]);
        return;
    }
    for (int i = tid; i < p.clusters * kHeadDim; i += kThreads) {
        if (cnt_s[i / kHeadDim] > 0) {
            const long long v = static_cast<long long>(hi_s[i]) * 1048576LL + lo_s[i];
            atomicAdd(reinterpret_cast<unsigned long long*>(sums_g + i), static_cast<unsigned long long>(v));
        }
    }
    for (int c = tid; c < p.clusters; c += kThreads)
        if (cnt_s[c] > 0) atomicAdd(&p.counts[unit * p.clusters + c], cnt_s[c]);
}

// ---- tcgen05 form of the assignment kernel (up to 32 centres) ---------------------------------------------------
// One CTA per SM; the 128-token tiles of all units are laid end to end and every CTA streams an equal share of them,
// segment by segment (a segment = consecutive tiles of one unit).  A tile arrives by two tensor-map copies
// (TMA, 128-byte swizzle: coordinates 0..63 and 64..127 of 128 rows) and is used three times without ever
// passing through registers:
//   * distances: D[128 tokens x 64] = X . [c_hi | c_lo]^T, X as the K-major A operand of tcgen05.mma, the centre
//     halves as a K-major B operand written once per segment; accumulator in TMEM, triple buffered;
//   * ranking: one thread per token (TMEM lane = token row) reads its row of D with tcgen05.ld, ranks the centres,
//     re-ranks near-ties exactly - only the centres inside the bound, with the arithmetic and order of the exact
//     path of the mma.sync form -, writes the id and sets one element of a one-hot operand
//     onehot[32 clusters x 128 tokens]; three groups of four warps take the tiles in turn, so each has three tile
//     periods for its chain of dependent steps;
//   * sums: S^T[128 coordinates x 32 clusters] += X^T . onehot^T, the same tile now read as the MN-major A operand,
//     accumulated in TMEM (four accumulators in turn) over the segment and flushed at its end as 2^24-scaled
//     integers.
// Three more warps issue the asynchronous work (distance MMAs, sum MMAs, copies); they stay converged (descriptor
// arithmetic on the uniform datapath) and elect one lane per instruction.  The roles run concurrently on
// different tiles and hand over through mbarriers only (triple-buffered distances and one-hot operands); every
// wait is bounded.
constexpr int kUGroups = 3;                    // token-owning groups; group g takes the tiles i = g (mod 3)
constexpr int kUGroupWarps = 4;                // a group: one warp per 32 token rows (TMEM lane quarter)
constexpr int kUThreads = (kUGroups * kUGroupWarps + 3) * 32;  // + three issuing warps: distance MMAs, sum MMAs, copies
constexpr int kUTile = 128;
constexpr int kUStages = 5;
constexpr int kUBoxBytes = kUTile * 128;       // 128 rows x 64 coordinates
constexpr int kUTileBytes = 2 * kUBoxBytes;
constexpr int kUOneHotBytes = 2 * 32 * 128;    // [2 token halves][32 clusters][64 tokens] FP16
constexpr uint32_t kUTmemCols = 512;           // distances 3 x 64 columns, sums 4 x 32 columns; a power of two
constexpr uint32_t kUColD = 0, kUColS = 192;
constexpr int kUSumBuffers = 4;                // tile i adds to accumulator i % 4: shorter FP32 chains, no MMA-to-MMA dependency
constexpr int kUChunkMax = 8192;               // most tokens per CTA (2048 per accumulator)

// Shared-memory matrix descriptor, 128-byte swizzle, address bits [4, 18), leading / stride byte offsets.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
           (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// FP16 x FP16 -> FP32, M = 128, N = n; a_mn: A is MN-major (the token tile read transposed).
__host__ __device__ constexpr uint32_t umma_idesc(int n, bool a_mn) {
    return (1u << 4) | (a_mn ? (1u << 15) : 0u) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One arrival on `bar` once every MMA issued so far by the calling thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Eight consecutive TMEM columns of the calling thread's lane (lane = 32 * (warp % 4) + lane id).
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&r)[8]) {
    uint32_t u[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7])
                 : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = __uint_as_float(u[i]);
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&r)[32]) {
    uint32_t u[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
          "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
          "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
          "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
        : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(u[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One box of a rank-3 tensor map (coordinate, token, unit) -> shared memory, completion counted on `bar`.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// Byte offset of 16-byte piece `piece` (0..7) of row `row` in a [rows][128 B] block with the 128-byte swizzle.
__device__ __forceinline__ uint32_t sw128(int row, int piece) { return row * 128 + ((piece ^ (row & 7)) << 4); }

// True in exactly one lane of a converged warp (the same lane every time).
__device__ __forceinline__ bool elect_one() {
    uint32_t chosen;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(chosen));
    return chosen != 0;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

constexpr int kUWorkers = kUThreads - 32;  // everyone but the copying warp: these meet at the segment boundaries

__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kUWorkers) : "memory"); }

template <bool HILO>
__global__ void __launch_bounds__(kUThreads, 1) kmeans_assign_umma_kernel(const KmeansParams p,
                                                                           const __grid_constant__ CUtensorMap xmap, int share,
                                                                           int first, int last) {
    extern __shared__ unsigned char smem_u[];
    constexpr int kN = HILO ? 64 : 32;  // rows of the centre operand: hi halves, then lo halves
    unsigned char* base = smem_u + ((1024u - (smem_u32(smem_u) & 1023u)) & 1023u);  // swizzled blocks: 1024-byte aligned
    unsigned char* xs = base;                                   // [stages][2 halves][128 tokens][128 B]
    unsigned char* cop = xs + kUStages * kUTileBytes;           // [2 halves][kN rows][128 B]
    unsigned char* oh = cop + 2 * kN * 128;                     // [groups][2 token halves][32 clusters][128 B]
    float* cen_s = reinterpret_cast<float*>(oh + kUGroups * kUOneHotBytes);  // [32][128] FP32 centres (exact re-ranking)
    float* cn_s = cen_s + 32 * kHeadDim;                        // [32] |c|^2, +inf for padding
    int* cnt_s = reinterpret_cast<int*>(cn_s + 32);             // [32]
    // full: tile landed (TMA bytes).  dist / sums: MMAs complete (tcgen05.commit); empty: the same event as sums,
    // counted per stage for the copying warp (a barrier of its own: no later completion can overtake its wait).
    // dist_free: the 128 threads of a group have read their distance buffer.  onehot: they have written their one-hot
    // operand.
    __shared__ uint64_t bar_full[kUStages], bar_empty[kUStages], bar_dist[kUGroups], bar_dist_free[kUGroups], bar_onehot[kUGroups],
        bar_sums[kUGroups];
    __shared__ uint32_t tmem_base_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Work of the launch = the tiles of all units laid end to end; CTA c takes [c * share, (c + 1) * share) and walks
    // it segment by segment (consecutive tiles of one unit, at most kUChunkMax tokens: one set of FP32 partial sums).
    // Tiles are numbered q = 0, 1, ... through the CTA's whole range: stage q % 5, group / distance buffer / one-hot
    // buffer q % 3, sum accumulator q % 4, and every barrier's phase follows from q, so the ring keeps turning across
    // segment boundaries (the copies of the next segment are in flight while this one drains and flushes).
    const int tiles_per_unit = (p.tokens + kUTile - 1) / kUTile;
    const long long work_total = static_cast<long long>(p.units) * tiles_per_unit;
    const long long work_begin = static_cast<long long>(blockIdx.x) * share;
    const long long work_end = work_begin + share < work_total ? work_begin + share : work_total;
    struct Segment {
        int unit, tile0, tiles;
    };
    auto segment_at = [&](long long w) {
        Segment sg;
        sg.unit = static_cast<int>(w / tiles_per_unit);
        sg.tile0 = static_cast<int>(w - static_cast<long long>(sg.unit) * tiles_per_unit);
        const long long left = work_end - w;
        sg.tiles = min(min(tiles_per_unit - sg.tile0, kUChunkMax / kUTile), static_cast<int>(left < 1 << 20 ? left : 1 << 20));
        return sg;
    };
    bool lost = false;

    if (tid == 0) {
        for (int s = 0; s < kUStages; ++s) mbar_init(&bar_full[s], 1), mbar_init(&bar_empty[s], 1);
        for (int b = 0; b < kUGroups; ++b) {
            mbar_init(&bar_dist[b], 1), mbar_init(&bar_sums[b], 1);
            mbar_init(&bar_dist_free[b], kUGroupWarps * 32), mbar_init(&bar_onehot[b], kUGroupWarps * 32);
        }
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(kUTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i < kUGroups * kUOneHotBytes / 16; i += kUThreads) reinterpret_cast<uint4*>(oh)[i] = make_uint4(0, 0, 0, 0);
    tc_fence_before();
    __syncthreads();  // barriers initialised, TMEM allocated, one-hot buffers empty
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    constexpr int kWarpDist = kUGroups * kUGroupWarps, kWarpCopy = kWarpDist + 2;  // kWarpDist + 1 issues the sum MMAs

    if (warp == kWarpCopy) {
        // ---- copies, through all segments without a stop: the stage of tile q is free once the sums of tile
        // q - 5 have run (whole warp, one elected lane per tile) --------------------------------------------------
        int q = 0;
        for (long long w = work_begin; w < work_end;) {
            const Segment sg = segment_at(w);
            for (int i = 0; i < sg.tiles; ++i, ++q) {
                if (q >= kUStages) lost |= !mbar_wait(&bar_empty[q % kUStages], (q / kUStages - 1) & 1);
                unsigned char* dst = xs + (q % kUStages) * kUTileBytes;
                uint64_t* bar = &bar_full[q % kUStages];
                if (elect_one()) {
                    mbar_arrive_expect_tx(bar, kUTileBytes);
                    tma_load_3d(dst, &xmap, 0, (sg.tile0 + i) * kUTile, sg.unit, bar);
                    tma_load_3d(dst + kUBoxBytes, &xmap, 64, (sg.tile0 + i) * kUTile, sg.unit, bar);
                }
                __syncwarp();
            }
            w += sg.tiles;
        }
    } else {
        int q0 = 0;     // tiles of the earlier segments of this CTA
        int prev = -1;  // byte offset of the element this thread set in its group's one-hot buffer
        for (long long w = work_begin; w < work_end;) {
            const Segment sg = segment_at(w);
            const int unit = sg.unit, n_tiles = sg.tiles;
            const int t_begin = sg.tile0 * kUTile, t_end = min(p.tokens, t_begin + n_tiles * kUTile);
            const float* cen_g = p.centres + static_cast<size_t>(unit) * p.clusters * kHeadDim;
            // ---- per segment: centre operand (FP16 hi | lo rows, swizzled), FP32 centres, |c|^2 -------------------
            {
                // four coordinates per thread and step, all loads of a thread in flight together
                constexpr int kSteps = (32 * kHeadDim / 4 + kUWorkers - 1) / kUWorkers;
                float4 v[kSteps];
#pragma unroll
                for (int k = 0; k < kSteps; ++k) {
                    const int i4 = tid + k * kUWorkers;
                    v[k] = (i4 < 32 * kHeadDim / 4 && i4 / (kHeadDim / 4) < p.clusters) ? __ldg(reinterpret_cast<const float4*>(cen_g) + i4)
                                                                                          : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int k = 0; k < kSteps; ++k) {
                    const int i4 = tid + k * kUWorkers;
                    if (i4 >= 32 * kHeadDim / 4) break;
                    const int c = i4 / (kHeadDim / 4), d = (i4 % (kHeadDim / 4)) * 4;
                    reinterpret_cast<float4*>(cen_s)[i4] = v[k];
                    const __half2 h01 = __floats2half2_rn(v[k].x, v[k].y), h23 = __floats2half2_rn(v[k].z, v[k].w);
                    unsigned char* at = cop + (d >> 6) * (kN * 128) + ((d & 7) << 1);
                    *reinterpret_cast<uint2*>(at + sw128(c, (d & 63) >> 3)) =
                        make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
                    float2 f01 = __half22float2(h01), f23 = __half22float2(h23);  // what the MMA sees: hi (+ lo)
                    if (HILO) {
                        const __half2 l01 = __floats2half2_rn(v[k].x - f01.x, v[k].y - f01.y);
                        const __half2 l23 = __floats2half2_rn(v[k].z - f23.x, v[k].w - f23.y);
                        *reinterpret_cast<uint2*>(at + sw128(32 + c, (d & 63) >> 3)) =
                            make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
                        const float2 g01 = __half22float2(l01), g23 = __half22float2(l23);
                        f01.x += g01.x, f01.y += g01.y, f23.x += g23.x, f23.y += g23.y;
                    }
                    // |c|^2: the 32 threads of a warp hold one centre (the worker count is a multiple of 32)
                    float sq = fmaf(f01.x, f01.x, fmaf(f01.y, f01.y, fmaf(f23.x, f23.x, f23.y * f23.y)));
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(kFull, sq, off);
                    if (lane == 0) cn_s[c] = c < p.clusters ? sq : INFINITY;
                }
            }
            if (tid < 32) cnt_s[tid] = 0;
            proxy_fence();  // the operands written above are read by the tensor core (async proxy)
            workers_sync();
            float cmax = lane < p.clusters ? cn_s[lane] : 0.f;  // largest |c|^2, in every thread
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) cmax = fmaxf(cmax, __shfl_xor_sync(kFull, cmax, off));
            const __half* xu = p.x + static_cast<size_t>(unit) * p.x_stride * kHeadDim;

            if (warp < kWarpDist) {
                // ---- ranking: one thread per token; group g takes the tiles with q = g (mod 3), distance buffer g
                // and one-hot buffer g ---------------------------------------------------------------------------
                const int g = warp / kUGroupWarps, quarter = warp % kUGroupWarps, row_in_tile = quarter * 32 + lane;
                const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
                // |x|^2 of a token is the same in every Lloyd iteration: the first one forms it and stores it (as FP32
                // bits) where the token's id goes, the following ones read it from there one tile of the group ahead,
                // the last one writes the id
                int32_t* ids_u = p.ids + static_cast<size_t>(unit) * p.tokens;
                const int i_first = (g + kUGroups - q0 % kUGroups) % kUGroups;
                float xn_next = 0.f;
                if (!first && t_begin + i_first * kUTile + row_in_tile < t_end)
                    xn_next = __int_as_float(ids_u[t_begin + i_first * kUTile + row_in_tile]);
                for (int i = i_first; i < n_tiles; i += kUGroups) {
                    const int q = q0 + i, use = q / kUGroups, st = q % kUStages;
                    const int row = t_begin + i * kUTile + row_in_tile;
                    const bool live = row < t_end;
                    float xn = xn_next;
                    if (!first && row + kUGroups * kUTile < t_end) xn_next = __int_as_float(ids_u[row + kUGroups * kUTile]);
                    lost |= !mbar_wait(&bar_dist[g], use & 1);
                    tc_fence_after();
                    float d[32];
                    tmem_ld32(tmem + lane_base + kUColD + g * 64, d);
                    if constexpr (HILO) {
                        float lo[32];
                        tmem_ld32(tmem + lane_base + kUColD + g * 64 + 32, lo);
                        tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 32; ++c) d[c] += lo[c];
                    } else {
                        tmem_ld_wait();
                    }
                    tc_fence_before();
                    mbar_arrive(&bar_dist_free[g]);  // the next distances of this group may be issued
                    float d1 = INFINITY, d2 = INFINITY;
                    int c1 = 0;
#pragma unroll
                    for (int c = 0; c < 32; ++c) {  // branch-free: best, second best, index of the best
                        d[c] = fmaf(-2.f, d[c], cn_s[c]);
                        d2 = fminf(d2, fmaxf(d[c], d1));
                        c1 = d[c] < d1 ? c : c1;  // a strict comparison keeps the lower index on ties
                        d1 = fminf(d1, d[c]);
                    }
                    if (first) {
                        // |x|^2 for the near-tie bound: packed FP16 products, eight at a time (an overflow gives +inf:
                        // re-rank)
                        lost |= !mbar_wait(&bar_full[st], (q / kUStages) & 1);
                        const unsigned char* xt = xs + st * kUTileBytes;
                        xn = 0.f;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const uint4 v = *reinterpret_cast<const uint4*>(xt + (j >> 3) * kUBoxBytes + sw128(row_in_tile, j & 7));
                            const __half2* h = reinterpret_cast<const __half2*>(&v);
                            __half2 s = __hmul2(h[0], h[0]);
                            s = __hfma2(h[1], h[1], s), s = __hfma2(h[2], h[2], s), s = __hfma2(h[3], h[3], s);
                            const float2 f = __half22float2(s);
                            xn += f.x + f.y;
                        }
                    }
                    // near-ties: only a centre whose distance lies inside the bound can win; the warp forms the exact
                    // FP32 sums of those few (same arithmetic, same order as `nearest`), one tied token at a time
                    const float bound = kTieBound * (1.01f * xn + cmax);
                    uint32_t inside = 0u;
                    if (live && !((d2 - d1) > bound)) {
#pragma unroll
                        for (int c = 0; c < 32; ++c) inside |= !((d[c] - d1) > bound) ? 1u << c : 0u;
                    }
                    uint32_t redo = __ballot_sync(kFull, inside != 0u);
                    while (redo) {
                        const int src = __ffs(redo) - 1;
                        redo &= redo - 1;
                        uint32_t cands = __shfl_sync(kFull, inside, src) & (p.clusters >= 32 ? 0xffffffffu : (1u << p.clusters) - 1u);
                        const __half* xr = xu + static_cast<size_t>(t_begin + i * kUTile + quarter * 32 + src) * kHeadDim;
                        float xv[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) xv[k] = __half2float(xr[lane + 32 * k]);
                        float best = INFINITY;
                        int bc = 0;
                        while (cands) {  // ascending centre index: the lower one wins ties
                            const int c = __ffs(cands) - 1;
                            cands &= cands - 1;
                            const float* crow = cen_s + c * kHeadDim;
                            float acc = 0.f;
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float df = xv[e] - crow[lane + 32 * e];
                                acc = fmaf(df, df, acc);
                            }
#pragma unroll
                            for (int off = 16; off > 0; off >>= 1) acc = acc + __shfl_xor_sync(kFull, acc, off);
                            if (acc < best) best = acc, bc = c;
                        }
                        if (lane == src) c1 = bc;
                    }
                    if (live) {
                        if (last) {
                            ids_u[row] = c1;
                        } else if (first) {
                            ids_u[row] = __float_as_int(xn);
                        }
                        atomicAdd(&cnt_s[c1], 1);
                    }
                    // one-hot buffer g was last read by the sums of tile q - 3
                    if (q >= kUGroups) lost |= !mbar_wait(&bar_sums[g], (use - 1) & 1);
                    unsigned char* ob = oh + g * kUOneHotBytes;
                    if (prev >= 0) *reinterpret_cast<unsigned short*>(ob + prev) = 0;
                    prev = -1;
                    if (live) {
                        prev = (row_in_tile >> 6) * (32 * 128) + sw128(c1, (row_in_tile & 63) >> 3) + ((row_in_tile & 7) << 1);
                        *reinterpret_cast<unsigned short*>(ob + prev) = 0x3C00;  // 1.0
                    }
                    proxy_fence();  // the tensor core (async proxy) reads what this thread wrote
                    mbar_arrive(&bar_onehot[g]);
                }
            } else if (warp == kWarpDist) {
                // ---- distance MMAs (whole warp, one elected lane per tile): tile q goes to buffer q % 3 as soon as
                // the group has read tile q - 3 out of it ----------------------------------------------------------
                const uint64_t a0 = umma_desc(smem_u32(xs), 16, 1024), b0 = umma_desc(smem_u32(cop), 16, 1024);
                for (int i = 0; i < n_tiles; ++i) {
                    const int q = q0 + i, buf = q % kUGroups;
                    if (q >= kUGroups) lost |= !mbar_wait(&bar_dist_free[buf], (q / kUGroups - 1) & 1);
                    lost |= !mbar_wait(&bar_full[q % kUStages], (q / kUStages) & 1);
                    tc_fence_after();
                    const uint64_t a = a0 + static_cast<uint64_t>(((q % kUStages) * kUTileBytes) >> 4);
                    const uint32_t d = tmem + kUColD + buf * 64;
                    if (elect_one()) {  // the eight MMAs and their commit in one elected stretch
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks) {  // 16 coordinates per step: 32 bytes inside the swizzled 128-byte row
                            const uint64_t ak = a + static_cast<uint64_t>(((ks >> 2) * kUBoxBytes + (ks & 3) * 32) >> 4);
                            const uint64_t bk = b0 + static_cast<uint64_t>(((ks >> 2) * (kN * 128) + (ks & 3) * 32) >> 4);
                            umma_f16(d, ak, bk, umma_idesc(kN, false), ks > 0);
                        }
                        umma_commit(&bar_dist[buf]);
                    }
                    __syncwarp();
                }
            } else {
                // ---- sum MMAs: the first four tiles of a segment start the four accumulators ----------------------
                const uint64_t a0 = umma_desc(smem_u32(xs), kUBoxBytes, 1024);  // MN-major: other half of the coordinates at LBO
                const uint64_t b0 = umma_desc(smem_u32(oh), 16, 1024);
                for (int i = 0; i < n_tiles; ++i) {
                    const int q = q0 + i, buf = q % kUGroups;
                    const uint64_t a = a0 + static_cast<uint64_t>(((q % kUStages) * kUTileBytes) >> 4);
                    const uint64_t o = b0 + static_cast<uint64_t>((buf * kUOneHotBytes) >> 4);
                    const uint32_t d = tmem + kUColS + (q % kUSumBuffers) * 32;
                    lost |= !mbar_wait(&bar_onehot[buf], (q / kUGroups) & 1);
                    tc_fence_after();
                    if (elect_one()) {
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks) {  // 16 tokens per step: two 8-row groups of the tile = 2048 bytes
                            const uint64_t ak = a + static_cast<uint64_t>((ks * 2048) >> 4);
                            const uint64_t bk = o + static_cast<uint64_t>(((ks >> 2) * (32 * 128) + (ks & 3) * 32) >> 4);
                            umma_f16(d, ak, bk, umma_idesc(32, true), (i >= kUSumBuffers || ks > 0) ? 1u : 0u);
                        }
                        umma_commit(&bar_sums[buf]);
                        umma_commit(&bar_empty[q % kUStages]);
                    }
                    __syncwarp();
                }
            }
            // ---- end of the segment: its sums go out (the commit of the last sum MMAs covers all of them) -----------
            const bool flusher = warp < 2 * kUGroupWarps;  // groups 0 and 1: coordinate row_in_tile, sixteen clusters each
            if (flusher) {
                const int q_last = q0 + n_tiles - 1;
                lost |= !mbar_wait(&bar_sums[q_last % kUGroups], (q_last / kUGroups) & 1);
                tc_fence_after();
            }
            workers_sync();
            if (flusher) {
                const int half = warp / kUGroupWarps, quarter = warp % kUGroupWarps, row_in_tile = quarter * 32 + lane;
                const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
                long long* sums_g = p.sums + static_cast<size_t>(unit) * p.clusters * kHeadDim;
#pragma unroll
                for (int part = 0; part < 2; ++part) {
                    float sum[8];  // the accumulators added in the order they were started
                    tmem_ld8(tmem + lane_base + kUColS + (q0 % kUSumBuffers) * 32 + 16 * half + 8 * part, sum);
                    tmem_ld_wait();
                    for (int a = 1; a < kUSumBuffers && a < n_tiles; ++a) {
                        float more[8];
                        tmem_ld8(tmem + lane_base + kUColS + ((q0 + a) % kUSumBuffers) * 32 + 16 * half + 8 * part, more);
                        tmem_ld_wait();
#pragma unroll
                        for (int k = 0; k < 8; ++k) sum[k] += more[k];
                    }
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const int c = 16 * half + 8 * part + k;
                        if (c < p.clusters && cnt_s[c] > 0)
                            atomicAdd(reinterpret_cast<unsigned long long*>(sums_g + c * kHeadDim + row_in_tile),
                                      static_cast<unsigned long long>(__float2ll_rn(sum[k] * kFix)));
                    }
                }
            }
            if (tid < p.clusters && cnt_s[tid] > 0) atomicAdd(&p.counts[unit * p.clusters + tid], cnt_s[tid]);
            tc_fence_before();
            workers_sync();  // accumulators, counters and the centre tables are free for the next segment
            tc_fence_after();
            q0 += n_tiles;
            w += n_tiles;
        }
    }
    if (lost) atomicOr(p.status, RESKV_STATUS_WAIT_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kUTmemCols) : "memory");
}

// New centres from the exact sums; clears sums and counts for the next round.
// `final_out` (FP16 [units, C, 128]) is written when non-null.
__global__ void kmeans_update_kernel(KmeansParams p, int value, __half* final_out) {
    const int unit = blockIdx.x;
    for (int i = threadIdx.x; i < p.clusters * kHeadDim; i += blockDim.x) {
        const size_t g = static_cast<size_t>(unit) * p.clusters * kHeadDim + i;
        const int n = p.counts[unit * p.clusters + i / kHeadDim];
        float c = p.centres[g];
        if (n > 0) {
            // exact integer sum / count, one rounding to FP32
            c = static_cast<float>(static_cast<double>(p.sums[g]) * (1.0 / 16777216.0) / static_cast<double>(n));
        } else if (value) {
            c = 0.f;
        }
        if (value) c = __half2float(__float2half_rn(c));
        p.centres[g] = c;
        p.sums[g] = 0;
        if (final_out) final_out[g] = __float2half_rn(c);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < p.clusters; c += blockDim.x) p.counts[unit * p.clusters + c] = 0;
}

// Decode-time step: grid (units, parts).  Optionally appends the mean of the group's tokens as centre
// `old_clusters`, then assigns the tokens.  Every CTA of a unit forms the same mean (the same additions in the
// same order); part 0 writes the new table; the tokens are assigned in `parts` contiguous slices, so that a
// small batch still fills the machine.
__global__ void __launch_bounds__(kThreads) kmeans_incremental_kernel(const __half* x, int64_t x_stride,
                                                                      const __half* old_cen, int old_clusters,
                                                                      __half* new_cen, int new_clusters, int tokens,
                                                                      int32_t* ids) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* cen_s = reinterpret_cast<float*>(smem);  // [new_clusters][128]
    const int unit = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool writer = blockIdx.y == 0;
    const __half* xg = x + static_cast<size_t>(unit) * x_stride * kHeadDim;
    for (int i = tid; i < old_clusters * kHeadDim; i += kThreads) {
        const __half v = old_cen[static_cast<size_t>(unit) * old_clusters * kHeadDim + i];
        cen_s[i] = __half2float(v);
        if (writer) new_cen[static_cast<size_t>(unit) * new_clusters * kHeadDim + i] = v;
    }
    if (new_clusters > old_clusters && tid < kHeadDim) {
        // mean of the group, FP32 accumulation in token order, rounded to FP16; the loads of eight tokens are
        // requested together, the additions stay sequential
        float s = 0.f;
        int t = 0;
        for (; t + 8 <= tokens; t += 8) {
            __half v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = xg[static_cast<size_t>(t + u) * kHeadDim + tid];
#pragma unroll
            for (int u = 0; u < 8; ++u) s += __half2float(v[u]);
        }
        for (; t < tokens; ++t) s += __half2float(xg[static_cast<size_t>(t) * kHeadDim + tid]);
        const __half m = __float2half_rn(s / static_cast<float>(tokens));
        cen_s[old_clusters * kHeadDim + tid] = __half2float(m);
        if (writer) new_cen[(static_cast<size_t>(unit) * new_clusters + old_clusters) * kHeadDim + tid] = m;
    }
    __syncthreads();
    const int per = (tokens + gridDim.y - 1) / gridDim.y;
    const int t_end = min(tokens, static_cast<int>(blockIdx.y + 1) * per);
    for (int t = blockIdx.y * per + warp; t < t_end; t += kWarps) {
        float xv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) xv[i] = __half2float(xg[static_cast<size_t>(t) * kHeadDim + lane + 32 * i]);
        float best;
        int c;
        nearest(cen_s, new_clusters, xv, lane, best, c);
        if (lane == 0) ids[static_cast<size_t>(unit) * tokens + t] = c;
    }
}

// torch.linspace(0, t-1, count).long(): float32 steps formed with a fused
// multiply-add, symmetric about the midpoint, truncated.
void linspace_indices(int t, int count, int* out) {
    if (count == 1) {
        out[0] = 0;
        return;
    }
    const float step = static_cast<float>(t - 1) / static_cast<float>(count - 1);
    for (int i = 0; i < count; ++i) {
        const double v = i < count / 2 ? static_cast<double>(step) * i
                                       : static_cast<double>(t - 1) - static_cast<double>(step) * (count - 1 - i);
        out[i] = static_cast<int>(static_cast<float>(v));
    }
}

// sums, centres, counts, then 256 bytes whose first word is the status word
size_t kmeans_ws_bytes(int units, int clusters) {
    const size_t per = static_cast<size_t>(units) * clusters;
    return per * kHeadDim * (sizeof(float) + sizeof(long long)) + per * sizeof(int) + 256;
}

using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                       const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up once through the runtime (no link against libcuda).
TensorMapEncodeFn tensor_map_encoder() {
    static const TensorMapEncodeFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &found) != cudaSuccess ||
            found != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<TensorMapEncodeFn>(f);
    }();
    return fn;
}

template <bool HILO>
int launch_umma(const KmeansParams& p, int value, int iterations, void* centroids, cudaStream_t s) {
    TensorMapEncodeFn encode = tensor_map_encoder();
    if (!encode) return fail(RESKV_ERR_CUDA, "kmeans: the driver offers no cuTensorMapEncodeTiled");
    // x as (coordinate, token, unit): boxes of 64 coordinates x 128 tokens, 128-byte swizzle, zeros beyond the
    // last token of a unit
    CUtensorMap xmap;
    const cuuint64_t dims[3] = {kHeadDim, static_cast<cuuint64_t>(p.tokens), static_cast<cuuint64_t>(p.units)};
    const cuuint64_t strides[2] = {kHeadDim * sizeof(__half), static_cast<cuuint64_t>(p.x_stride) * kHeadDim * sizeof(__half)};
    const cuuint32_t box[3] = {64, kUTile, 1}, elem[3] = {1, 1, 1};
    const CUresult made = encode(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(p.x), dims, strides, box, elem,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (made != CUDA_SUCCESS) return fail(RESKV_ERR_CUDA, "kmeans: cuTensorMapEncodeTiled failed with code %d", static_cast<int>(made));
    constexpr int kN = HILO ? 64 : 32;
    const size_t smem = 1024 + static_cast<size_t>(kUStages) * kUTileBytes + 2 * kN * 128 + kUGroups * kUOneHotBytes +
                        32 * kHeadDim * sizeof(float) + 32 * (sizeof(float) + sizeof(int));
    static unsigned long long prepared = 0;  // per-device bit: the shared-memory attribute is set
    int dev = 0;
    cudaGetDevice(&dev);
    if (!((prepared >> (dev & 63)) & 1ull)) {
        if (int rc = check_cuda(cudaFuncSetAttribute(kmeans_assign_umma_kernel<HILO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     static_cast<int>(smem)),
                                "cudaFuncSetAttribute(kmeans_assign_umma)"))
            return rc;
        prepared |= 1ull << (dev & 63);
    }
    // One CTA per SM, every CTA an equal share of all units' tiles.  A CTA pays about ten tile times per segment
    // (pipeline drain, flush, new centre tables, refill), so the share is chosen - between the even split and
    // half as much again - for the shortest slowest CTA: a share that divides the units evenly often beats the
    // smallest one.
    const int tiles_unit = (p.tokens + kUTile - 1) / kUTile, seg_max = kUChunkMax / kUTile;
    const long long tiles_total = static_cast<long long>(p.units) * tiles_unit;
    const long long even = (tiles_total + sm_count() - 1) / sm_count();
    long long share = even < 4 ? 4 : even, best_cost = -1;
    for (long long cand = share; cand <= share + share / 2 + 1; ++cand) {
        long long worst = 0;
        for (long long w0 = 0; w0 < tiles_total; w0 += cand) {
            const long long w1 = w0 + cand < tiles_total ? w0 + cand : tiles_total;
            long long segments = 0;
            for (long long w = w0; w < w1;) {  // same walk as the kernel's
                const long long in_unit = tiles_unit - w % tiles_unit;
                long long n = in_unit < w1 - w ? in_unit : w1 - w;
                if (n > seg_max) n = seg_max;
                w += n, ++segments;
            }
            const long long cost = (w1 - w0) + 10 * segments;
            if (cost > worst) worst = cost;
        }
        if (best_cost < 0 || worst < best_cost) best_cost = worst, share = cand;
    }
    const dim3 grid(static_cast<unsigned>((tiles_total + share - 1) / share));
    for (int it = 0; it < iterations; ++it) {
        kmeans_assign_umma_kernel<HILO><<<grid, kUThreads, smem, s>>>(p, xmap, static_cast<int>(share), it == 0, it + 1 == iterations);
        kmeans_update_kernel<<<p.units, 256, 0, s>>>(p, value, it + 1 == iterations ? static_cast<__half*>(centroids) : nullptr);
    }
    return check_cuda(cudaGetLastError(), "kmeans launch");
}

}  // namespace
}  // namespace reskv

using namespace reskv;

extern "C" size_t reskv_kmeans_workspace_bytes(int batch, int kv_heads, int clusters) {
    if (batch < 1 || kv_heads < 1 || clusters < 1 || clusters > kMaxClusters) return 0;
    return kmeans_ws_bytes(batch * kv_heads, clusters);
}

extern "C" int reskv_kmeans(const void* x, int batch, int kv_heads, int tokens, int64_t x_tok_stride, int clusters,
                            int iterations, int value, void* workspace, size_t workspace_bytes, void* centroids,
                            int32_t* ids, void* stream) {
    if (!x || !centroids || !ids) return fail(RESKV_ERR_INVALID, "kmeans: null tensor pointer");
    if (batch < 1 || kv_heads < 1 || tokens < 1) return fail(RESKV_ERR_INVALID, "kmeans: batch, heads and tokens must be positive");
    if (clusters < 1 || clusters > kMaxClusters) return fail(RESKV_ERR_INVALID, "kmeans: cluster count must be in [1,64], got %d", clusters);
    if (iterations < 1) return fail(RESKV_ERR_INVALID, "kmeans: iterations must be positive");
    if (x_tok_stride < tokens) return fail(RESKV_ERR_INVALID, "kmeans: token stride smaller than token count");
    const int units = batch * kv_heads;
    const size_t need = kmeans_ws_bytes(units, clusters);
    if (!workspace || workspace_bytes < need)
        return fail(RESKV_ERR_WORKSPACE, "kmeans: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    if (int rc = check_device_pointer(x, "kmeans", "x")) return rc;
    if (int rc = check_device_pointer(centroids, "kmeans", "centroids")) return rc;
    const size_t per = static_cast<size_t>(units) * clusters * kHeadDim;
    KmeansParams p{};
    p.x = static_cast<const __half*>(x);
    p.sums = static_cast<long long*>(workspace);  // 8-byte aligned first
    p.centres = reinterpret_cast<float*>(p.sums + per);
    p.counts = reinterpret_cast<int*>(p.centres + per);
    p.status = reinterpret_cast<uint32_t*>(p.counts + static_cast<size_t>(units) * clusters);
    p.ids = ids;
    p.x_stride = x_tok_stride;
    p.units = units, p.tokens = tokens, p.clusters = clusters;
    InitIndex init{};
    if (tokens >= clusters) {
        linspace_indices(tokens, clusters, init.idx);
    } else {
        // fewer tokens than centres: every token once, then tokens repeated in order
        for (int c = 0; c < clusters; ++c) init.idx[c] = c % tokens;
    }
    // `value`: bit 0 = V flavour, bit 1 = exact (integer) accumulation of the cluster sums, bit 2 = the mma.sync
    // form of the tensor-core sums instead of the tcgen05 one
    const bool exact = (value & 2) != 0, warp_mma = (value & 4) != 0;
    value &= 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    kmeans_init_kernel<<<units, 256, 0, s>>>(p, init, value);
    const int padded = (clusters + 7) / 8 * 8;
    // the integer-counter arrays double as the FP32 reduction buffer [32][kRedStride] of the tensor-core form
    size_t counters = static_cast<size_t>(clusters) * kHeadDim * 2 * sizeof(int);
    const bool fast = !exact && padded <= 32 && aligned16(x);  // the row staging copies 16-byte pieces
    if (fast && !warp_mma && aligned16(workspace)) return value ? launch_umma<false>(p, value, iterations, centroids, s) : launch_umma<true>(p, value, iterations, centroids, s);
    if (fast) counters = static_cast<size_t>(kWarps) * 32 * kRedStride * sizeof(float);
    const size_t smem = static_cast<size_t>(clusters) * kHeadDim * sizeof(float) + counters +
                        kMaxClusters * (sizeof(int) + sizeof(float)) +
                        static_cast<size_t>(padded) * kCenHalfStride * sizeof(__half) * (value ? 1 : 2) +
                        (fast ? static_cast<size_t>(kWarps) * 16 * kXsRow : 0);
    void (*kernel)(const KmeansParams, int, int) =
        fast ? (value ? kmeans_assign_mma_kernel<false, true> : kmeans_assign_mma_kernel<true, true>)
             : (value ? kmeans_assign_mma_kernel<false, false> : kmeans_assign_mma_kernel<true, false>);
    if (smem > 48 * 1024) {
        if (int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)),
                                "cudaFuncSetAttribute(kmeans_assign)"))
            return rc;
    }
    // tensor-core form: as many tokens per CTA as still leave about two CTAs per SM (set-up and the final
    // reduction are per CTA), between kChunk and kChunkFastMax
    int chunk = kChunk;
    if (fast) {
        const long long want = static_cast<long long>(units) * tokens / (2ll * sm_count());
        chunk = static_cast<int>(want < kChunk ? kChunk : want > kChunkFastMax ? kChunkFastMax : (want + 127) / 128 * 128);
    }
    const dim3 grid((tokens + chunk - 1) / chunk, units);
    for (int it = 0; it < iterations; ++it) {
        kernel<<<grid, kThreads, smem, s>>>(p, padded, chunk);
        kmeans_update_kernel<<<units, 256, 0, s>>>(p, value, it + 1 == iterations ? static_cast<__half*>(centroids) : nullptr);
    }
    return check_cuda(cudaGetLastError(), "kmeans launch");
}

extern "C" int reskv_kmeans_status(const void* workspace, int batch, int kv_heads, int clusters, uint32_t* status, void* stream) {
    if (!workspace || !status) return fail(RESKV_ERR_INVALID, "kmeans_status: null pointer");
    if (batch < 1 || kv_heads < 1 || clusters < 1 || clusters > kMaxClusters) return fail(RESKV_ERR_INVALID, "kmeans_status: bad sizes");
    const size_t per = static_cast<size_t>(batch) * kv_heads * clusters;
    const size_t at = per * kHeadDim * (sizeof(float) + sizeof(long long)) + per * sizeof(int);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (int rc = check_cuda(cudaMemcpyAsync(status, static_cast<const unsigned char*>(workspace) + at, sizeof(uint32_t),
                                            cudaMemcpyDeviceToHost, s),
                            "kmeans_status copy"))
        return rc;
    return check_cuda(cudaStreamSynchronize(s), "kmeans_status synchronize");
}

extern "C" int reskv_kmeans_incremental(const void* x, int batch, int kv_heads, int tokens, int64_t x_tok_stride,
                                        const void* old_centroids, int old_clusters, void* new_centroids,
                                        int new_clusters, int32_t* ids, void* stream) {
    if (!x || !old_centroids || !new_centroids || !ids) return fail(RESKV_ERR_INVALID, "kmeans_incremental: null tensor pointer");
    if (int rc = check_device_pointer(x, "kmeans_incremental", "x")) return rc;
    if (int rc = check_device_pointer(new_centroids, "kmeans_incremental", "new_centroids")) return rc;
    if (batch < 1 || kv_heads < 1 || tokens < 1) return fail(RESKV_ERR_INVALID, "kmeans_incremental: batch, heads and tokens must be positive");
    if (old_clusters < 1 || new_clusters > kMaxClusters || (new_clusters != old_clusters && new_clusters != old_clusters + 1))
        return fail(RESKV_ERR_INVALID, "kmeans_incremental: centre counts must satisfy 1 <= old <= new <= old + 1 <= 64");
    if (x_tok_stride < tokens) return fail(RESKV_ERR_INVALID, "kmeans_incremental: token stride smaller than token count");
    const size_t smem = static_cast<size_t>(new_clusters) * kHeadDim * sizeof(float);
    // slices of the group per unit: enough CTAs for one per SM, at least one warp-load of tokens each
    int parts = 1;
    while (parts < 8 && batch * kv_heads * parts < sm_count() && tokens >= 2 * kWarps * parts) parts *= 2;
    kmeans_incremental_kernel<<<dim3(batch * kv_heads, parts), kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), x_tok_stride, static_cast<const __half*>(old_centroids), old_clusters,
        static_cast<__half*>(new_centroids), new_clusters, tokens, ids);
    return check_cuda(cudaGetLastError(), "kmeans_incremental launch");
}

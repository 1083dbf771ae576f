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

// Decode-time step: one CTA per unit.  Optionally appends the mean of the
// group's tokens as centre `old_clusters`, then assigns the tokens.
__global__ void __launch_bounds__(kThreads) kmeans_incremental_kernel(const __half* x, int64_t x_stride,
                                                                      const __half* old_cen, int old_clusters,
                                                                      __half* new_cen, int new_clusters, int tokens,
                                                                      int32_t* ids) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* cen_s = reinterpret_cast<float*>(smem);  // [new_clusters][128]
    const int unit = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const __half* xg = x + static_cast<size_t>(unit) * x_stride * kHeadDim;
    for (int i = tid; i < old_clusters * kHeadDim; i += kThreads) {
        const __half v = old_cen[static_cast<size_t>(unit) * old_clusters * kHeadDim + i];
        cen_s[i] = __half2float(v);
        new_cen[static_cast<size_t>(unit) * new_clusters * kHeadDim + i] = v;
    }
    if (new_clusters > old_clusters && tid < kHeadDim) {
        // mean of the group, FP32 accumulation in token order, rounded to FP16
        float s = 0.f;
        for (int t = 0; t < tokens; ++t) s += __half2float(xg[static_cast<size_t>(t) * kHeadDim + tid]);
        const __half m = __float2half_rn(s / static_cast<float>(tokens));
        cen_s[old_clusters * kHeadDim + tid] = __half2float(m);
        new_cen[(static_cast<size_t>(unit) * new_clusters + old_clusters) * kHeadDim + tid] = m;
    }
    __syncthreads();
    for (int t = warp; t < tokens; t += kWarps) {
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

size_t kmeans_ws_bytes(int units, int clusters) {
    const size_t per = static_cast<size_t>(units) * clusters;
    return per * kHeadDim * (sizeof(float) + sizeof(long long)) + per * sizeof(int) + 256;
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
    // `value`: bit 0 = V flavour, bit 1 = exact (integer) accumulation of the cluster sums
    const bool exact = (value & 2) != 0;
    value &= 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    kmeans_init_kernel<<<units, 256, 0, s>>>(p, init, value);
    const int padded = (clusters + 7) / 8 * 8;
    // the integer-counter arrays double as the FP32 reduction buffer [32][kRedStride] of the tensor-core form
    size_t counters = static_cast<size_t>(clusters) * kHeadDim * 2 * sizeof(int);
    const bool fast = !exact && padded <= 32 && aligned16(x);  // the row staging copies 16-byte pieces
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
    kmeans_incremental_kernel<<<batch * kv_heads, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), x_tok_stride, static_cast<const __half*>(old_centroids), old_clusters,
        static_cast<__half*>(new_centroids), new_clusters, tokens, ids);
    return check_cuda(cudaGetLastError(), "kmeans_incremental launch");
}

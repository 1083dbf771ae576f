// Fused split-K decode attention over the unstructured FP16 bitmap layout, with
// deferred value-centroid fusion.
//
// For a query q, compressed keys k_t = ck[idk_t] + rk_t and values
// v_t = cv[idv_t] + rv_t (rk, rv sparse, stored as bitmap + packed FP16):
//
//   s_t  = scaling * < R(pos_q) q , R(start + t) k_t >          (half-split RoPE)
//   out  = sum_t p_t v_t / sum_t p_t
//        = ( sum_t p_t rv_t  +  sum_c beta_c cv[c] ) / l ,  beta_c = sum_{idv_t = c} p_t
//
// so the token loop only touches residuals and accumulates the per-cluster mass
// beta; the value centroids are applied once, after the split-K reduction
// (same decomposition as the reference, cluster_mass.cu:3-11).
//
// Kernel 1 (partial): grid (splits, units).  A CTA streams its token range in
// tiles of 64 tokens.  Bitmaps and payloads of a tile are contiguous in global
// memory, so each tile is four 1-D bulk copies (TMA) into a shared-memory ring,
// completion tracked by one mbarrier per stage.  Each warp owns every eighth
// token of a tile; a lane owns coordinates {l, l+32, l+64, l+96}, which keeps
// both RoPE partners (d, d+64) in one lane.  A kept coordinate's payload index
// is the popcount of the bitmap bits above it.  The key is rotated once and
// shared by all query heads of the KV head (GQA); RoPE sin/cos advance by a
// fixed rotation per token and are re-seeded every 16 tiles.
//
// Kernel 2 (merge): one CTA per query head reduces the split partials, applies
// the value centroids, and -- when a dense recent window is given -- folds its
// tokens into the same softmax.
#include "decode_common.cuh"

namespace reskv {
namespace {

// Sum GQA per-lane partials over the warp; every lane ends with all totals.
template <int GQA>
__device__ __forceinline__ void warp_sum_heads(float (&v)[GQA], int lane) {
    if constexpr (GQA == 4) {
        const bool up = lane & 16;
        float send0 = up ? v[0] : v[2], send1 = up ? v[1] : v[3];
        float keep0 = up ? v[2] : v[0], keep1 = up ? v[3] : v[1];
        keep0 += __shfl_xor_sync(0xffffffffu, send0, 16);
        keep1 += __shfl_xor_sync(0xffffffffu, send1, 16);
        const bool up2 = lane & 8;
        float send = up2 ? keep0 : keep1;
        float y = (up2 ? keep1 : keep0) + __shfl_xor_sync(0xffffffffu, send, 8);
        y += __shfl_xor_sync(0xffffffffu, y, 4);
        y += __shfl_xor_sync(0xffffffffu, y, 2);
        y += __shfl_xor_sync(0xffffffffu, y, 1);
        // lanes [0,8) hold head 0, [8,16) head 1, [16,24) head 2, [24,32) head 3
#pragma unroll
        for (int h = 0; h < 4; ++h) v[h] = __shfl_sync(0xffffffffu, y, h * 8);
    } else {
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v[h] += __shfl_xor_sync(0xffffffffu, v[h], off);
        }
    }
}

// ---- residual layouts --------------------------------------------------------------------
// A layout says how many payload / metadata bytes a token has and how a lane
// turns them into the residual of its four coordinates {lane + 32 i}.

// Unstructured FP16: 2 x u64 bitmap, MSB first (reference compression.py:84-88).
// Words in memory order: x = word0 low half (coords 32..63), y = word0 high half
// (0..31), z = word1 low (96..127), w = word1 high (64..95); inside a 32-bit half
// coordinate c sits at bit 31 - c % 32; payload index = retained coordinates before it.
template <int NNZ>
struct LayoutBitmap {
    static constexpr int kPayloadBytes = NNZ * 2, kMetaBytes = 16;
    static constexpr bool kScale = false;
    __device__ static void decode(const unsigned char* pay, const unsigned char* meta, float, int lane,
                                  float (&r)[4]) {
        const uint4 bm = *reinterpret_cast<const uint4*>(meta);
        const __half* row = reinterpret_cast<const __half*>(pay);
        const uint32_t word[4] = {bm.y, bm.x, bm.w, bm.z};
        int base = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = word[i];
            const int rank = base + __popc(__funnelshift_rc(w, 0u, 32 - lane));
            const bool kept = (w >> (31 - lane)) & 1u;
            r[i] = kept ? __half2float(row[min(rank, NNZ - 1)]) : 0.0f;
            base += __popc(w);
        }
    }
};

// Unstructured INT4 / INT2: every coordinate stored, value i of a word at bit
// i * BITS, two's complement, times the token's scale (reference.py:16-20).
template <int BITS>
struct LayoutQuant {
    static constexpr int kPayloadBytes = 16 * BITS, kMetaBytes = 0;
    static constexpr bool kScale = true;
    __device__ static void decode(const unsigned char* pay, const unsigned char*, float scale, int lane,
                                  float (&r)[4]) {
        constexpr int kPer = 32 / BITS, kSign = 1 << (BITS - 1);
        const uint32_t* w = reinterpret_cast<const uint32_t*>(pay);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = lane + 32 * i;
            const int c = (w[d / kPer] >> ((d % kPer) * BITS)) & ((1 << BITS) - 1);
            r[i] = static_cast<float>((c ^ kSign) - kSign) * scale;
        }
    }
};

// Tiled FP16 (STRUCT = false): one 16-bit LSB-first mask per 16-wide tile, values
// in (tile, ascending coordinate) order.  4:16 structured FP16 (STRUCT = true):
// four 4-bit in-tile indices per tile (reference.py:37-48).  Metadata word i
// carries tile 2i in its low and tile 2i+1 in its high half.
template <int NNZ, bool STRUCT>
struct LayoutTiled {
    static constexpr int kPayloadBytes = NNZ * 2, kMetaBytes = 16;
    static constexpr bool kScale = false;
    __device__ static void decode(const unsigned char* pay, const unsigned char* meta, float, int lane,
                                  float (&r)[4]) {
        const uint4 mw = *reinterpret_cast<const uint4*>(meta);
        const __half* row = reinterpret_cast<const __half*>(pay);
        const uint32_t word[4] = {mw.x, mw.y, mw.z, mw.w};
        const int local = lane & 15, shift = lane & 16;
        constexpr int kPerTile = NNZ / 8;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t code = (word[i] >> shift) & 0xffffu;
            const int tile = 2 * i + (lane >> 4);
            float v = 0.f;
            if constexpr (STRUCT) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (((code >> (4 * k)) & 15u) == static_cast<uint32_t>(local)) v = __half2float(row[tile * 4 + k]);
            } else {
                if ((code >> local) & 1u) v = __half2float(row[tile * kPerTile + __popc(code & ((1u << local) - 1u))]);
            }
            r[i] = v;
        }
    }
};

// 1-of-4 structured INT4: 32 signed nibbles + 32 two-bit in-group indices
// (reference.py:27-36).
struct LayoutStructInt4 {
    static constexpr int kPayloadBytes = 16, kMetaBytes = 8;
    static constexpr bool kScale = true;
    __device__ static void decode(const unsigned char* pay, const unsigned char* meta, float scale, int lane,
                                  float (&r)[4]) {
        const uint4 pw = *reinterpret_cast<const uint4*>(pay);
        const uint2 mw = *reinterpret_cast<const uint2*>(meta);
        const uint32_t packed[4] = {pw.x, pw.y, pw.z, pw.w};
        const uint32_t m[2] = {mw.x, mw.y};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int gi = 8 * i + (lane >> 2);
            const uint32_t sel = (m[gi >> 4] >> (2 * (gi & 15))) & 3u;
            const int nib = (packed[gi >> 3] >> (4 * (gi & 7))) & 15;
            r[i] = (sel == static_cast<uint32_t>(lane & 3)) ? static_cast<float>((nib ^ 8) - 8) * scale : 0.f;
        }
    }
};

template <class L>
struct Stage {
    alignas(16) unsigned char kp[kTile * L::kPayloadBytes];
    alignas(16) unsigned char vp[kTile * L::kPayloadBytes];
    alignas(16) unsigned char km[kTile * (L::kMetaBytes ? L::kMetaBytes : 1)];
    alignas(16) unsigned char vm[kTile * (L::kMetaBytes ? L::kMetaBytes : 1)];
};

// Warp-per-token partial kernel, generic over the residual layout.
template <int GQA, class L, int CVS>
__global__ void __launch_bounds__(kThreads, 2) decode_simt_partial_kernel(const DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int kStages = (sizeof(Stage<L>) <= 10240) ? 4 : 3;
    // metadata rows that are not a multiple of 16 bytes cannot be bulk-copied at every
    // token offset: such metadata is copied by the threads themselves
    constexpr bool kMetaBulk = (L::kMetaBytes % 16) == 0;
    using StageT = Stage<L>;
    StageT* stages = reinterpret_cast<StageT*>(smem_raw);
    __half* kc_s = reinterpret_cast<__half*>(smem_raw + sizeof(StageT) * kStages);
    __shared__ uint64_t full_bar[kStages];
    __shared__ float red_m[GQA][kWarps];
    __shared__ float red_l[GQA][kWarps];
    __shared__ uint32_t timed_out;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, unit = blockIdx.y;
    const int b = unit / p.kh, hkv = unit % p.kh;

    const int tokens = token_count(p);
    const int total_tiles = (tokens + kTile - 1) / kTile;
    const int per_split = split_tiles(p, total_tiles);
    const int tile_begin = split * per_split;
    const int tile_end = min(total_tiles, tile_begin + per_split);
    const int ntiles = max(0, tile_end - tile_begin);

    const size_t unit_tok = static_cast<size_t>(unit) * p.tok_stride;
    const unsigned char* kp_g = static_cast<const unsigned char*>(p.kp) + unit_tok * L::kPayloadBytes;
    const unsigned char* vp_g = static_cast<const unsigned char*>(p.vp) + unit_tok * L::kPayloadBytes;
    const unsigned char* km_g = static_cast<const unsigned char*>(p.kb) + unit_tok * L::kMetaBytes;
    const unsigned char* vm_g = static_cast<const unsigned char*>(p.vb) + unit_tok * L::kMetaBytes;
    const int8_t* kid_g = p.kid + unit_tok;
    const int8_t* vid_g = p.vid + unit_tok;
    const __half* ks_g = L::kScale ? p.ks + unit_tok : nullptr;
    const __half* vs_g = L::kScale ? p.vs + unit_tok : nullptr;

    if (tid == 0) {
        timed_out = 0;
        for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    auto issue = [&](int tile_rel) {
        // one thread: bulk copies of tile `tile_rel` into its ring slot
        const int t0 = (tile_begin + tile_rel) * kTile;
        const int n = min(kTile, tokens - t0);
        StageT& st = stages[tile_rel % kStages];
        uint64_t* bar = &full_bar[tile_rel % kStages];
        const uint32_t pl_bytes = n * L::kPayloadBytes;
        const uint32_t md_bytes = (kMetaBulk && L::kMetaBytes) ? n * L::kMetaBytes : 0u;
        mbar_arrive_expect_tx(bar, 2 * pl_bytes + 2 * md_bytes);
        bulk_g2s(st.kp, kp_g + static_cast<size_t>(t0) * L::kPayloadBytes, pl_bytes, bar);
        bulk_g2s(st.vp, vp_g + static_cast<size_t>(t0) * L::kPayloadBytes, pl_bytes, bar);
        if (md_bytes) {
            bulk_g2s(st.km, km_g + static_cast<size_t>(t0) * L::kMetaBytes, md_bytes, bar);
            bulk_g2s(st.vm, vm_g + static_cast<size_t>(t0) * L::kMetaBytes, md_bytes, bar);
        }
    };
    auto copy_meta = [&](int tile_rel) {
        // all threads: metadata of tile `tile_rel` with plain 4-byte loads
        if constexpr (!kMetaBulk && L::kMetaBytes > 0) {
            if (tile_rel >= ntiles) return;
            const int t0 = (tile_begin + tile_rel) * kTile;
            const int words = min(kTile, tokens - t0) * (L::kMetaBytes / 4);
            StageT& st = stages[tile_rel % kStages];
            const uint32_t* ksrc = reinterpret_cast<const uint32_t*>(km_g + static_cast<size_t>(t0) * L::kMetaBytes);
            const uint32_t* vsrc = reinterpret_cast<const uint32_t*>(vm_g + static_cast<size_t>(t0) * L::kMetaBytes);
            for (int i = tid; i < words; i += kThreads) {
                reinterpret_cast<uint32_t*>(st.km)[i] = __ldg(ksrc + i);
                reinterpret_cast<uint32_t*>(st.vm)[i] = __ldg(vsrc + i);
            }
        }
    };
    if (tid == 0) {
        for (int s = 0; s < kStages && s < ntiles; ++s) issue(s);
    }
    for (int s = 0; s < kStages; ++s) copy_meta(s);

    // key centroid table -> shared memory (FP16, as stored)
    {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.kc + static_cast<size_t>(unit) * p.ck * kHeadDim);
        uint32_t* dst = reinterpret_cast<uint32_t*>(kc_s);
        for (int i = tid; i < p.ck * kHeadDim / 2; i += kThreads) dst[i] = __ldg(src + i);
    }

    // query, rotated at pos_q, pre-multiplied by scaling * log2(e)
    const float f0 = rope_freq(p.inv_freq, p.theta, lane);
    const float f1 = rope_freq(p.inv_freq, p.theta, lane + 32);
    float qr[GQA][4];
    {
        float s0, c0, s1, c1;
        const float pq = static_cast<float>(query_position(p));
        sincosf(pq * f0, &s0, &c0);
        sincosf(pq * f1, &s1, &c1);
        const float mul = p.scaling * kLog2e;
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
            const __half* qh = p.q + (static_cast<size_t>(b) * p.nh + hkv * GQA + h) * kHeadDim;
            const float a0 = __half2float(qh[lane]), a1 = __half2float(qh[lane + 32]);
            const float a2 = __half2float(qh[lane + 64]), a3 = __half2float(qh[lane + 96]);
            qr[h][0] = (a0 * c0 - a2 * s0) * mul;
            qr[h][2] = (a2 * c0 + a0 * s0) * mul;
            qr[h][1] = (a1 * c1 - a3 * s1) * mul;
            qr[h][3] = (a3 * c1 + a1 * s1) * mul;
        }
    }
    // fixed rotation between consecutive tokens of this warp (kWarps positions)
    float ds0, dc0, ds1, dc1;
    sincosf(static_cast<float>(kWarps) * f0, &ds0, &dc0);
    sincosf(static_cast<float>(kWarps) * f1, &ds1, &dc1);

    float m_run[GQA], l_run[GQA], acc[GQA][4], bet[GQA][CVS];
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[h][i] = 0.f;
#pragma unroll
        for (int i = 0; i < CVS; ++i) bet[h][i] = 0.f;
    }

    // ids (and scales) of this warp's tokens in the next tile, one token per lane < kTokPerWarp
    auto load_ids = [&](int tile_rel, int& kid, int& vid, float& ksc, float& vsc) {
        kid = vid = 0;
        ksc = vsc = 0.f;
        const int t = (tile_begin + tile_rel) * kTile + warp + kWarps * lane;
        if (tile_rel < ntiles && lane < kTokPerWarp && t < tokens) {
            kid = kid_g[t];
            vid = vid_g[t];
            if constexpr (L::kScale) {
                ksc = __half2float(ks_g[t]);
                vsc = __half2float(vs_g[t]);
            }
        }
    };
    int kid_next, vid_next;
    float ksc_next, vsc_next;
    load_ids(0, kid_next, vid_next, ksc_next, vsc_next);
    __syncthreads();  // centroid table (and hand-copied metadata) ready

    float rs0 = 0.f, rc0 = 1.f, rs1 = 0.f, rc1 = 1.f;
    bool lost = false;
    for (int it = 0; it < ntiles; ++it) {
        const int t0 = (tile_begin + it) * kTile;
        const int kid_cur = kid_next, vid_cur = vid_next;
        const float ksc_cur = ksc_next, vsc_cur = vsc_next;
        load_ids(it + 1, kid_next, vid_next, ksc_next, vsc_next);
        if (it % kReseedTiles == 0) {
            const float pos = static_cast<float>(p.start_pos + t0 + warp);
            sincosf(pos * f0, &rs0, &rc0);
            sincosf(pos * f1, &rs1, &rc1);
        }
        if (!mbar_wait(&full_bar[it % kStages], (it / kStages) & 1)) lost = true;
        const StageT& st = stages[it % kStages];
#pragma unroll 2
        for (int j = 0; j < kTokPerWarp; ++j) {
            const int tl = warp + kWarps * j;  // token within the tile
            if (t0 + tl < tokens) {
                const int kid = __shfl_sync(0xffffffffu, kid_cur, j);
                const int vid = __shfl_sync(0xffffffffu, vid_cur, j);
                float ksc = 0.f, vsc = 0.f;
                if constexpr (L::kScale) {
                    ksc = __shfl_sync(0xffffffffu, ksc_cur, j);
                    vsc = __shfl_sync(0xffffffffu, vsc_cur, j);
                }
                float kv[4], vr[4];
                L::decode(st.kp + tl * L::kPayloadBytes, st.km + tl * L::kMetaBytes, ksc, lane, kv);
                L::decode(st.vp + tl * L::kPayloadBytes, st.vm + tl * L::kMetaBytes, vsc, lane, vr);
                const __half* crow = kc_s + min(max(kid, 0), p.ck - 1) * kHeadDim;
                kv[0] += __half2float(crow[lane]);
                kv[1] += __half2float(crow[lane + 32]);
                kv[2] += __half2float(crow[lane + 64]);
                kv[3] += __half2float(crow[lane + 96]);
                const float k0 = kv[0] * rc0 - kv[2] * rs0, k2 = kv[2] * rc0 + kv[0] * rs0;
                const float k1 = kv[1] * rc1 - kv[3] * rs1, k3 = kv[3] * rc1 + kv[1] * rs1;
                float s[GQA];
#pragma unroll
                for (int h = 0; h < GQA; ++h)
                    s[h] = qr[h][0] * k0 + qr[h][1] * k1 + qr[h][2] * k2 + qr[h][3] * k3;
                warp_sum_heads<GQA>(s, lane);
#pragma unroll
                for (int h = 0; h < GQA; ++h) {
                    const float m_new = fmaxf(m_run[h], s[h]);
                    const float corr = fast_exp2(m_run[h] - m_new);
                    const float pr = fast_exp2(s[h] - m_new);
                    m_run[h] = m_new;
                    l_run[h] = l_run[h] * corr + pr;
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[h][i] = acc[h][i] * corr + pr * vr[i];
#pragma unroll
                    for (int i = 0; i < CVS; ++i)
                        bet[h][i] = bet[h][i] * corr + ((lane + 32 * i == vid) ? pr : 0.f);
                }
            }
            // advance this warp's RoPE state by kWarps positions
            const float ns0 = rs0 * dc0 + rc0 * ds0, nc0 = rc0 * dc0 - rs0 * ds0;
            const float ns1 = rs1 * dc1 + rc1 * ds1, nc1 = rc1 * dc1 - rs1 * ds1;
            rs0 = ns0, rc0 = nc0, rs1 = ns1, rc1 = nc1;
        }
        __syncthreads();  // every warp is done with this ring slot
        if (tid == 0 && it + kStages < ntiles) issue(it + kStages);
        copy_meta(it + kStages);
    }
    if (lost && lane == 0) atomicOr(&timed_out, 1u);

    // ---- combine the warps of the CTA ------------------------------------------
    if (lane == 0) {
#pragma unroll
        for (int h = 0; h < GQA; ++h) red_m[h][warp] = m_run[h], red_l[h][warp] = l_run[h];
    }
    __syncthreads();
    // stage buffers are free now: reuse them for the cross-warp sums
    float* red_acc = reinterpret_cast<float*>(smem_raw);               // [kWarps][GQA][128]
    float* red_bet = red_acc + kWarps * GQA * kHeadDim;                // [kWarps][GQA][32*CVS]
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
        float fm = red_m[h][0];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) fm = fmaxf(fm, red_m[h][w]);
        const float sc = (m_run[h] == -INFINITY) ? 0.f : fast_exp2(m_run[h] - fm);
#pragma unroll
        for (int i = 0; i < 4; ++i) red_acc[(warp * GQA + h) * kHeadDim + lane + 32 * i] = acc[h][i] * sc;
#pragma unroll
        for (int i = 0; i < CVS; ++i) red_bet[(warp * GQA + h) * (32 * CVS) + lane + 32 * i] = bet[h][i] * sc;
    }
    __syncthreads();
    const size_t part = static_cast<size_t>(b) * p.nh + hkv * GQA;  // first query head of this unit
    for (int idx = tid; idx < GQA * kHeadDim; idx += kThreads) {
        const int h = idx / kHeadDim, d = idx % kHeadDim;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) sum += red_acc[(w * GQA + h) * kHeadDim + d];
        p.ws_delta[((part + h) * p.splits + split) * kHeadDim + d] = sum;
    }
    for (int idx = tid; idx < GQA * 32 * CVS; idx += kThreads) {
        const int h = idx / (32 * CVS), c = idx % (32 * CVS);
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) sum += red_bet[(w * GQA + h) * (32 * CVS) + c];
        p.ws_beta[((part + h) * p.splits + split) * kMaxClusters + c] = sum;
    }
    if (tid < GQA) {
        const int h = tid;
        float fm = red_m[h][0];
        for (int w = 1; w < kWarps; ++w) fm = fmaxf(fm, red_m[h][w]);
        float fl = 0.f;
        for (int w = 0; w < kWarps; ++w)
            fl += (red_m[h][w] == -INFINITY) ? 0.f : red_l[h][w] * fast_exp2(red_m[h][w] - fm);
        p.ws_m[(part + h) * p.splits + split] = fm;  // log2 domain
        p.ws_l[(part + h) * p.splits + split] = fl;
    }
    if (tid == 0 && timed_out) atomicOr(p.status, RESKV_STATUS_WAIT_TIMEOUT);
}

#include "decode_mma.cuh"

// ---- merge -----------------------------------------------------------------------
struct MergeParams {
    const float* ws_m;      // log2-domain maxima [BNH][splits], or natural-log m [BNH] when splits == 0
    const float* ws_l;
    const float* ws_delta;
    const float* ws_beta;
    const __half* vc;       // [B*KH,CV,128]
    const __half* comp_out; // splits == 0: finished compressed result to merge with
    const __half* rq;       // rotated query [BNH,128] or null
    const __half* rk;       // rotated recent keys [B*KH,Tr,128] or null
    const __half* rv;       // recent values
    const float* rscores;   // precomputed scaled scores [BNH,Tr] (natural units) or null
    __half* out;
    float* out_m;
    float* out_l;
    int kh, nh, splits, cv, tr;
    float scaling;
    const int32_t* dyn;  // device step state: dyn[1] = recent tokens (overrides tr), or null
    int recent_cap;      // tokens between units in rk / rv (== tr for contiguous windows)
    uint32_t* status;    // device status word of the call's workspace, or null
};

constexpr int kMergeThreads = 128;
constexpr int kMaxRecent = 1024;  // recent tokens whose scores fit the shared buffer
constexpr int kRecentChunk = 32;  // recent tokens staged in shared memory at a time

// rows x 128 FP16 values, global -> shared, 16 bytes per thread and copy (all in flight at once)
__device__ __forceinline__ void stage_rows(__half* dst, const __half* src, int rows, int tid, int threads) {
    for (int i = tid; i < rows * (kHeadDim / 8); i += threads) cp_async16(dst + i * 8, src + i * 8);
}

// dynamic shared memory of the merge kernel: value centroids, one chunk of recent keys and of recent
// values (shared by the unit's query heads), recent scores per head
constexpr int kMergePartStride = kHeadDim + kMaxClusters + 4;
size_t merge_smem_bytes(int cv, int gqa, int recent_max) {
    return (static_cast<size_t>(cv) + 2 * kRecentChunk) * kHeadDim * sizeof(__half) +
           static_cast<size_t>(gqa) * ((kMergeThreads / 32) * kMergePartStride + (recent_max + 3) / 4 * 4) * sizeof(float);
}

// One CTA per (sequence, KV head) unit, 128 threads per query head of the unit; thread (h, d) owns
// output coordinate d of head h.  Everything that is read with a stride or by several heads (value
// centroids, recent keys and values) is staged in shared memory by 16-byte asynchronous copies
// issued up front, so the kernel pays a few memory round trips instead of one per centroid and
// per recent token.
__global__ void __launch_bounds__(1024) decode_merge_kernel(const MergeParams p, int recent_max) {
    extern __shared__ __align__(16) unsigned char merge_smem[];
    __shared__ float beta_s[8][kMaxClusters];
    __shared__ float red[8][kMergeThreads / 32];
    constexpr int kPartStride = kMergePartStride;  // per (head, warp): delta, cluster masses, max, sum
    const int gqa = p.nh / p.kh, threads = gqa * kMergeThreads;
    const int unit = blockIdx.x, tid = threadIdx.x;
    const int h = tid / kMergeThreads, d = tid % kMergeThreads, lane = d & 31, warp = d >> 5;
    const int fq = unit * gqa + h;  // (b * kh + hkv) * gqa + h == b * nh + hkv * gqa + h
    const int sc_stride = (recent_max + 3) / 4 * 4;
    __half* vc_s = reinterpret_cast<__half*>(merge_smem);
    __half* rk_s = vc_s + static_cast<size_t>(p.cv) * kHeadDim;
    __half* rv_s = rk_s + kRecentChunk * kHeadDim;
    float* part_s = reinterpret_cast<float*>(rv_s + kRecentChunk * kHeadDim);  // [gqa][4 warps][kPartStride]
    float* sc_s = part_s + gqa * (kMergeThreads / 32) * kPartStride + h * sc_stride;
    const int tr = p.dyn ? min(p.dyn[1], recent_max) : p.tr;
    // a window count beyond the buffers is cut (the newest tokens are then missing from the result): tell the host
    if (p.dyn && p.status && tid == 0 && unit == 0 && (p.dyn[1] > recent_max || p.dyn[1] < 0))
        atomicOr(p.status, RESKV_STATUS_STATE_RANGE);
    const bool dot_scores = tr > 0 && !p.rscores;
    const __half* rk_g = p.rk ? p.rk + static_cast<size_t>(unit) * p.recent_cap * kHeadDim : nullptr;
    const __half* rv_g = p.rv ? p.rv + static_cast<size_t>(unit) * p.recent_cap * kHeadDim : nullptr;

    // group 0: value centroids + first chunk of recent keys; group 1: first chunk of recent values
    if (p.splits > 0) stage_rows(vc_s, p.vc + static_cast<size_t>(unit) * p.cv * kHeadDim, p.cv, tid, threads);
    if (dot_scores) stage_rows(rk_s, rk_g, min(tr, kRecentChunk), tid, threads);
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (tr > 0) stage_rows(rv_s, rv_g, min(tr, kRecentChunk), tid, threads);
    asm volatile("cp.async.commit_group;" ::: "memory");

    // rotated query of this head, requested together with everything else the kernel reads
    float qv[4] = {0.f, 0.f, 0.f, 0.f};
    if (dot_scores) {
        const __half* qrow = p.rq + static_cast<size_t>(fq) * kHeadDim;
#pragma unroll
        for (int i = 0; i < 4; ++i) qv[i] = __half2float(qrow[lane + 32 * i]);
    }

    // compressed part: numerator `num`, max `m2` (log2 domain), sum `l`
    float m2, l, num;
    if (p.splits > 0) {
        // The four warps of a head share the splits (warp w takes splits w, w + 4, ...) and read each
        // partial row with 16-byte loads (lane: coordinates 4 lane .. 4 lane + 3; lanes 0..15 also four
        // cluster masses), so all loads of a warp are in flight together; the four partial results are
        // combined through shared memory.
        const float* pm = p.ws_m + static_cast<size_t>(fq) * p.splits;
        const float* pl = p.ws_l + static_cast<size_t>(fq) * p.splits;
        float wm = -INFINITY;
        for (int s = warp; s < p.splits; s += kMergeThreads / 32) wm = fmaxf(wm, pm[s]);
        float wl = 0.f;
        float4 wn = make_float4(0.f, 0.f, 0.f, 0.f), wb = wn;
#pragma unroll 4
        for (int s = warp; s < p.splits; s += kMergeThreads / 32) {
            if (pm[s] == -INFINITY) continue;  // empty slot: its delta / beta rows were never written
            const float w = fast_exp2(pm[s] - wm);
            const size_t row = static_cast<size_t>(fq) * p.splits + s;
            const float4 dv = *reinterpret_cast<const float4*>(p.ws_delta + row * kHeadDim + 4 * lane);
            wl += pl[s] * w;
            wn.x += dv.x * w, wn.y += dv.y * w, wn.z += dv.z * w, wn.w += dv.w * w;
            if (lane < kMaxClusters / 4) {
                const float4 bv = *reinterpret_cast<const float4*>(p.ws_beta + row * kMaxClusters + 4 * lane);
                wb.x += bv.x * w, wb.y += bv.y * w, wb.z += bv.z * w, wb.w += bv.w * w;
            }
        }
        float* slot = part_s + (h * (kMergeThreads / 32) + warp) * kPartStride;  // [delta 128 | beta 64 | m | l]
        *reinterpret_cast<float4*>(slot + 4 * lane) = wn;
        if (lane < kMaxClusters / 4) *reinterpret_cast<float4*>(slot + kHeadDim + 4 * lane) = wb;
        if (lane == 0) slot[kHeadDim + kMaxClusters] = wm, slot[kHeadDim + kMaxClusters + 1] = wl;
        __syncthreads();
        const float* mine = part_s + h * (kMergeThreads / 32) * kPartStride;
        m2 = -INFINITY;
#pragma unroll
        for (int w = 0; w < kMergeThreads / 32; ++w) m2 = fmaxf(m2, mine[w * kPartStride + kHeadDim + kMaxClusters]);
        l = 0.f, num = 0.f;
        float bsum = 0.f;
#pragma unroll
        for (int w = 0; w < kMergeThreads / 32; ++w) {
            const float* ps = mine + w * kPartStride;
            const float pmw = ps[kHeadDim + kMaxClusters];
            const float sc = (pmw == -INFINITY) ? 0.f : fast_exp2(pmw - m2);
            l += ps[kHeadDim + kMaxClusters + 1] * sc;
            num += ps[d] * sc;
            if (d < p.cv) bsum += ps[kHeadDim + d] * sc;
        }
        if (d < kMaxClusters) beta_s[h][d] = (d < p.cv) ? bsum : 0.f;
        if (d == 0) {
            if (p.out_m) p.out_m[fq] = m2 * kLn2;
            if (p.out_l) p.out_l[fq] = l;
        }
    } else {
        m2 = p.ws_m[fq] * kLog2e;
        l = p.ws_l[fq];
        num = __half2float(p.comp_out[static_cast<size_t>(fq) * kHeadDim + d]) * l;
    }
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();  // beta_s, vc_s and the first key chunk are in place
    if (p.splits > 0) {
#pragma unroll 8
        for (int c = 0; c < p.cv; ++c) num = fmaf(beta_s[h][c], __half2float(vc_s[c * kHeadDim + d]), num);
    }

    if (tr > 0) {
        // scores of the recent tokens (log2 domain) into shared memory
        if (p.rscores) {
            for (int t = d; t < tr; t += kMergeThreads)
                sc_s[t] = p.rscores[static_cast<size_t>(fq) * tr + t] * kLog2e;
        } else {
            const float mul = p.scaling * kLog2e;
            for (int c0 = 0; c0 < tr; c0 += kRecentChunk) {
                const int n = min(kRecentChunk, tr - c0);
                if (c0 > 0) {  // later chunks: plain staging, one round trip each
                    __syncthreads();
                    stage_rows(rk_s, rk_g + static_cast<size_t>(c0) * kHeadDim, n, tid, threads);
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                    __syncthreads();
                }
                for (int t = warp; t < n; t += kMergeThreads / 32) {
                    const __half* krow = rk_s + t * kHeadDim;
                    float dot = 0.f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) dot = fmaf(qv[i], __half2float(krow[lane + 32 * i]), dot);
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
                    if (lane == 0) sc_s[c0 + t] = dot * mul;
                }
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // scores and the first value chunk are in place
        float rm = -INFINITY;
        for (int t = d; t < tr; t += kMergeThreads) rm = fmaxf(rm, sc_s[t]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) rm = fmaxf(rm, __shfl_xor_sync(0xffffffffu, rm, off));
        if (lane == 0) red[h][warp] = rm;
        __syncthreads();
        rm = fmaxf(fmaxf(red[h][0], red[h][1]), fmaxf(red[h][2], red[h][3]));
        const float jm = fmaxf(rm, m2);
        const float cw = (m2 == -INFINITY) ? 0.f : fast_exp2(m2 - jm);
        float rnum = 0.f, rl = 0.f;
        for (int c0 = 0; c0 < tr; c0 += kRecentChunk) {
            const int n = min(kRecentChunk, tr - c0);
            if (c0 > 0) {
                __syncthreads();
                stage_rows(rv_s, rv_g + static_cast<size_t>(c0) * kHeadDim, n, tid, threads);
                asm volatile("cp.async.commit_group;" ::: "memory");
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                __syncthreads();
            }
#pragma unroll 8
            for (int t = 0; t < n; ++t) {
                const float w = fast_exp2(sc_s[c0 + t] - jm);
                rl += w;
                rnum = fmaf(w, __half2float(rv_s[t * kHeadDim + d]), rnum);
            }
        }
        num = num * cw + rnum;
        l = l * cw + rl;
    }
    p.out[static_cast<size_t>(fq) * kHeadDim + d] = __float2half_rn(num / fmaxf(l, 1e-20f));
}

// cudaFuncSetAttribute(max dynamic shared memory) once per kernel instance and device, not per call.
// `done` is a per-instantiation bit mask over device ordinals (< 64); a race between host threads only
// repeats the idempotent call.
template <class Kernel>
int allow_smem(Kernel kern, size_t smem, unsigned long long& done, const char* what) {
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    const bool tracked = dev >= 0 && dev < 64;
    if (tracked && (done >> dev & 1ull)) return RESKV_OK;
    if (int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)), what))
        return rc;
    if (tracked) done |= 1ull << dev;
    return RESKV_OK;
}

// one CTA per unit with 128 threads per query head of the unit
int launch_merge(const MergeParams& mp, int units, int recent_max, cudaStream_t s) {
    const int gqa = mp.nh / mp.kh;
    if (gqa < 1 || gqa > 8) return fail(RESKV_ERR_INVALID, "merge: at most 8 query heads per KV head");
    const size_t smem = merge_smem_bytes(mp.splits > 0 ? mp.cv : 0, gqa, recent_max);
    if (smem > 48 * 1024) {
        static unsigned long long done = 0;
        if (int rc = allow_smem(decode_merge_kernel, merge_smem_bytes(kMaxClusters, 8, kMaxRecent), done,
                                "cudaFuncSetAttribute(decode_merge)"))
            return rc;
    }
    decode_merge_kernel<<<units, gqa * kMergeThreads, smem, s>>>(mp, recent_max);
    return check_cuda(cudaGetLastError(), "decode_merge launch");
}

template <int GQA, class L, int CVS>
int launch_simt_cvs(const DecodeParams& p, int units, cudaStream_t stream) {
    constexpr int kStages = (sizeof(Stage<L>) <= 10240) ? 4 : 3;
    size_t smem = sizeof(Stage<L>) * kStages + static_cast<size_t>(p.ck) * kHeadDim * sizeof(__half);
    const size_t red_bytes = static_cast<size_t>(kWarps) * GQA * (kHeadDim + 32 * CVS) * sizeof(float);
    if (smem < red_bytes) smem = red_bytes;
    auto kern = decode_simt_partial_kernel<GQA, L, CVS>;
    // the kernel's shared memory grows with the key centroid count: allow the maximum once
    static unsigned long long done = 0;
    const size_t smem_max = sizeof(Stage<L>) * kStages + static_cast<size_t>(kMaxClusters) * kHeadDim * sizeof(__half);
    if (int rc = allow_smem(kern, smem_max > red_bytes ? smem_max : red_bytes, done, "cudaFuncSetAttribute(decode_simt_partial)"))
        return rc;
    kern<<<dim3(p.splits, units), kThreads, smem, stream>>>(p);
    return check_cuda(cudaGetLastError(), "decode_simt_partial launch");
}

template <int GQA, class L>
int launch_simt(const DecodeParams& p, int units, cudaStream_t s) {
    return p.cv <= 32 ? launch_simt_cvs<GQA, L, 1>(p, units, s) : launch_simt_cvs<GQA, L, 2>(p, units, s);
}

template <int GQA, int NNZ, int BETA>
int launch_partial_mma_beta(const DecodeParams& p, cudaStream_t stream) {
    using ML = mma::LayoutMmaBitmap<NNZ>;
    const size_t smem = mma::smem_bytes<GQA, ML>(p.ck);
    auto kern = mma::decode_mma_kernel<GQA, ML, BETA>;
    static unsigned long long done = 0;
    if (int rc = allow_smem(kern, mma::smem_bytes<GQA, ML>(kMaxClusters), done, "cudaFuncSetAttribute(decode_bitmap_mma)"))
        return rc;
    kern<<<p.grid, mma::kThreadsM, smem, stream>>>(p);
    return check_cuda(cudaGetLastError(), "decode_bitmap_mma launch");
}

// up to 32 value centroids: the instance with two cluster-mass blocks
template <int GQA, int NNZ>
int launch_partial_mma(const DecodeParams& p, int, cudaStream_t stream) {
    return p.cv <= 32 ? launch_partial_mma_beta<GQA, NNZ, 2>(p, stream) : launch_partial_mma_beta<GQA, NNZ, 4>(p, stream);
}

// 0 = tensor-core kernel (default), 1 = warp-per-token SIMT kernel
int g_variant = 0;
// optional events recorded right before / after the partial kernel (profiling aid)
cudaEvent_t g_ev_start = nullptr, g_ev_stop = nullptr;

enum LayoutId { kBitmap32, kBitmap64, kQuant4, kQuant2, kTiled64, kStruct32, kStructInt4, kCompact4x64, kCompact4x32, kCompact2x64 };

template <int GQA>
int dispatch_layout(const DecodeParams& p, LayoutId layout, int units, cudaStream_t s) {
    switch (layout) {
        case kBitmap32:
            return g_variant == 0 ? launch_partial_mma<GQA, 32>(p, units, s) : launch_simt<GQA, LayoutBitmap<32>>(p, units, s);
        case kBitmap64:
            return g_variant == 0 ? launch_partial_mma<GQA, 64>(p, units, s) : launch_simt<GQA, LayoutBitmap<64>>(p, units, s);
        case kQuant4:
            return g_variant == 0 ? launch_packed_mma(p, 0, GQA, units, s) : launch_simt<GQA, LayoutQuant<4>>(p, units, s);
        case kQuant2:
            return g_variant == 0 ? launch_packed_mma(p, 1, GQA, units, s) : launch_simt<GQA, LayoutQuant<2>>(p, units, s);
        case kTiled64:
            return g_variant == 0 ? launch_packed_mma(p, 2, GQA, units, s)
                                  : launch_simt<GQA, LayoutTiled<64, false>>(p, units, s);
        case kStruct32:
            return g_variant == 0 ? launch_packed_mma(p, 3, GQA, units, s)
                                  : launch_simt<GQA, LayoutTiled<32, true>>(p, units, s);
        case kCompact4x64:
        case kCompact4x32:
        case kCompact2x64:
            if (g_variant != 0)
                return fail(RESKV_ERR_INVALID, "the compact quantised layout has no warp-per-token kernel");
            return launch_packed_mma(p, 5 + (layout - kCompact4x64), GQA, units, s);
        default: {
            // 8-byte metadata rows can only be bulk-copied when every tile starts 16-byte aligned
            const bool bulk_ok = p.tokens % 2 == 0 && p.tok_stride % 2 == 0 && aligned16(p.kb) && aligned16(p.vb);
            return (g_variant == 0 && bulk_ok) ? launch_packed_mma(p, 4, GQA, units, s)
                                               : launch_simt<GQA, LayoutStructInt4>(p, units, s);
        }
    }
}

int pick_splits(int units, int tokens) {
    const int tiles = (tokens + kTile - 1) / kTile;
    const int slots = sm_count() * 2;  // two CTAs per SM
    int best = 1;
    double best_cost = 1e30;
    const int max_splits = tiles < 64 ? tiles : 64;
    for (int s = 1; s <= max_splits; ++s) {
        const int per = (tiles + s - 1) / s;
        const int used = (tiles + per - 1) / per;  // splits that actually get tiles
        if (used != s) continue;
        const long ctas = static_cast<long>(units) * s;
        const long waves = (ctas + slots - 1) / slots;
        // time ~ waves * tiles per CTA, plus a per-split cost for the merge and CTA prologue
        const double cost = static_cast<double>(waves) * (per + 1.5) + 0.02 * s;
        if (cost < best_cost - 1e-9) best_cost = cost, best = s;
    }
    return best;
}

size_t workspace_bytes(int bnh, int splits) {
    const size_t rows = static_cast<size_t>(bnh) * splits;
    return kWsHeader + rows * (2 + kHeadDim + kMaxClusters) * sizeof(float);
}

// How a decode call is cut into partial results.
struct PartialPlan {
    int slots;     // partial results per query head in the workspace
    int chunk;     // tiles per CTA
    int grid;      // CTAs of the tensor-core kernel (the warp-per-token kernel runs slots x units)
    int balanced;  // 1: equal share of all tiles per CTA, 0: one CTA per (unit, split)
};

// splits_req > 0 (caller's choice) or the warp-per-token kernel: fixed splits per unit.  Otherwise the balanced
// schedule: at most two CTAs per SM, every CTA streams ceil(all tiles / CTAs) consecutive tiles, so the per-CTA
// tables are built once per CTA and no SM idles on a partial last wave.  A unit of n tiles is then touched by at
// most (n - 1) / chunk + 2 CTAs.  With a device-side token count (`dyn`) chunk is recomputed on the device as
// ceil(units * n / grid), which keeps that figure below ceil(grid / units) + 1 for any n.
PartialPlan plan_partials(int units, int tokens, int splits_req, bool tensor_core, bool dyn, int64_t tok_stride) {
    const int tiles = (tokens + kTile - 1) / kTile;
    PartialPlan pp{};
    if (splits_req > 0 || !tensor_core) {
        int splits = splits_req > 0 ? splits_req : pick_splits(units, tokens);
        if (splits > tiles) splits = tiles;
        const int per = (tiles + splits - 1) / splits;
        splits = (tiles + per - 1) / per;  // drop splits that would get no tile
        pp.slots = splits, pp.chunk = per, pp.grid = units * splits, pp.balanced = 0;
        return pp;
    }
    const long long max_tiles = dyn ? (tok_stride + kTile - 1) / kTile : tiles;
    const long long all = static_cast<long long>(units) * (dyn ? max_tiles : tiles);
    long long grid = static_cast<long long>(RESKV_MMA_CTAS_PER_SM) * sm_count();
    if (grid > all) grid = all;
    const long long chunk = (static_cast<long long>(units) * tiles + grid - 1) / grid;
    if (dyn) {
        pp.slots = static_cast<int>((grid + units - 1) / units) + 1;
    } else {
        grid = (static_cast<long long>(units) * tiles + chunk - 1) / chunk;  // CTAs that get tiles
        const long long s = (tiles - 1) / chunk + 2;
        pp.slots = static_cast<int>(s < tiles ? s : tiles);
    }
    pp.chunk = static_cast<int>(chunk), pp.grid = static_cast<int>(grid), pp.balanced = 1;
    return pp;
}

}  // namespace
}  // namespace reskv

using namespace reskv;

extern "C" int reskv_decode_set_variant(int variant) {
    if (variant != 0 && variant != 1) return fail(RESKV_ERR_INVALID, "decode_set_variant: 0 (tensor-core) or 1 (SIMT), got %d", variant);
    g_variant = variant;
    return RESKV_OK;
}

extern "C" int reskv_decode_set_timing_events(void* start, void* stop) {
    g_ev_start = static_cast<cudaEvent_t>(start);
    g_ev_stop = static_cast<cudaEvent_t>(stop);
    return RESKV_OK;
}

extern "C" int reskv_decode_auto_splits(int batch, int kv_heads, int tokens) {
    if (batch < 1 || kv_heads < 1 || tokens < 1) return fail(RESKV_ERR_INVALID, "auto_splits: sizes must be positive");
    return pick_splits(batch * kv_heads, tokens);
}

extern "C" size_t reskv_decode_bitmap_fp16_workspace_bytes(int batch, int kv_heads, int q_heads, int tokens,
                                                           int splits) {
    if (batch < 1 || kv_heads < 1 || q_heads < 1 || tokens < 1) return 0;
    // enough for either kernel variant and for a device-side token count (decode_step) up to `tokens`
    const int units = batch * kv_heads;
    int slots = plan_partials(units, tokens, splits, true, false, tokens).slots;
    const int a = plan_partials(units, tokens, splits, false, false, tokens).slots;
    const int b = plan_partials(units, tokens, splits, true, true, tokens).slots;
    if (a > slots) slots = a;
    if (b > slots) slots = b;
    return workspace_bytes(batch * q_heads, slots);
}

namespace {
struct DecodeArgs {
    const void *q, *kc, *kid, *kp, *km, *ks, *vc, *vid, *vp, *vm, *vs;
    int batch, kv_heads, q_heads, tokens;
    int64_t tok_stride;
    int ck, cv, start_pos, pos_q;
    float theta;
    const float* inv_freq;
    float scaling;
    int splits;
    const void *rq, *rk, *rv;
    int recent_tokens;
    void* workspace;
    size_t workspace_bytes;
    void* out;
    float *out_m, *out_l;
    void* stream;
    const int32_t* dyn = nullptr;  // device step state {pos_q, recent tokens}
    int recent_cap = 0;            // window capacity in tokens when dyn is given
    bool clear_status = false;     // zero the workspace's status header once the arguments are accepted
};

// Which partial kernel dispatch_layout will pick for this call (its partial plan differs).
bool tensor_core_variant(LayoutId layout, const DecodeArgs& a) {
    if (layout == kStructInt4) {
        const bool bulk_ok = a.tokens % 2 == 0 && a.tok_stride % 2 == 0 && aligned16(a.km) && aligned16(a.vm);
        return g_variant == 0 && bulk_ok;
    }
    if (layout == kCompact4x64 || layout == kCompact4x32 || layout == kCompact2x64) return true;
    return g_variant == 0;
}

int decode_common(const DecodeArgs& a, LayoutId layout, bool has_meta, bool has_scale, const char* who) {
    if (!a.q || !a.kc || !a.kid || !a.kp || !a.vc || !a.vid || !a.vp || !a.out)
        return fail(RESKV_ERR_INVALID, "%s: null tensor pointer", who);
    if (has_meta && (!a.km || !a.vm)) return fail(RESKV_ERR_INVALID, "%s: null metadata pointer", who);
    if (has_scale && (!a.ks || !a.vs)) return fail(RESKV_ERR_INVALID, "%s: null scale pointer", who);
    if (a.batch < 1 || a.kv_heads < 1 || a.q_heads < 1 || a.tokens < 1)
        return fail(RESKV_ERR_INVALID, "%s: batch, heads and tokens must be positive", who);
    if (a.q_heads % a.kv_heads) return fail(RESKV_ERR_INVALID, "%s: q_heads must be a multiple of kv_heads", who);
    const int gqa = a.q_heads / a.kv_heads;
    if (gqa != 1 && gqa != 4 && gqa != 8)
        return fail(RESKV_ERR_INVALID, "%s: supported query/kv head ratios are 1, 4 and 8, got %d", who, gqa);
    if (a.ck < 1 || a.ck > kMaxClusters || a.cv < 1 || a.cv > kMaxClusters)
        return fail(RESKV_ERR_INVALID, "%s: centroid counts must be in [1,64]", who);
    if (a.tok_stride < a.tokens) return fail(RESKV_ERR_INVALID, "%s: tok_stride < tokens", who);
    if (!a.dyn && a.pos_q < a.start_pos + a.tokens - 1)
        return fail(RESKV_ERR_INVALID, "%s: query position precedes compressed tokens", who);
    if (a.dyn && (a.recent_cap < 1 || a.recent_cap > kMaxRecent || !a.rq || !a.rk || !a.rv))
        return fail(RESKV_ERR_INVALID, "%s: a step state needs the window buffers and a capacity in [1,%d]", who, kMaxRecent);
    if (!aligned16(a.kp) || !aligned16(a.vp) || (has_meta && layout != kStructInt4 && (!aligned16(a.km) || !aligned16(a.vm))))
        return fail(RESKV_ERR_INVALID, "%s: payload and metadata pointers must be 16-byte aligned", who);
    if (!aligned16(a.kc) || !aligned16(a.vc) || (reinterpret_cast<uintptr_t>(a.q) & 1u))
        return fail(RESKV_ERR_INVALID, "%s: misaligned centroid (16 bytes) or query pointer", who);
    if ((a.rk && !aligned16(a.rk)) || (a.rv && !aligned16(a.rv)))
        return fail(RESKV_ERR_INVALID, "%s: recent keys and values must be 16-byte aligned", who);
    if (int rc = check_device_pointer(a.q, who, "q")) return rc;
    if (int rc = check_device_pointer(a.kp, who, "k_payload")) return rc;
    if (int rc = check_device_pointer(a.out, who, "out")) return rc;
    const bool has_recent = a.recent_tokens > 0;
    if (a.recent_tokens < 0 || (has_recent && (!a.rq || !a.rk || !a.rv)))
        return fail(RESKV_ERR_INVALID, "%s: recent window needs rotated q, rotated k and v", who);
    if (a.recent_tokens > kMaxRecent)
        return fail(RESKV_ERR_LIMIT, "%s: at most %d recent tokens, got %d", who, kMaxRecent, a.recent_tokens);

    const int units = a.batch * a.kv_heads;
    const PartialPlan pp = plan_partials(units, a.tokens, a.splits, tensor_core_variant(layout, a), a.dyn != nullptr, a.tok_stride);
    const int splits = pp.slots, per = pp.chunk;
    const size_t need = workspace_bytes(a.batch * a.q_heads, splits);
    if (!a.workspace || a.workspace_bytes < need)
        return fail(RESKV_ERR_WORKSPACE, "%s: workspace of %zu bytes needed, %zu given", who, need, a.workspace_bytes);

    if (a.clear_status) {
        if (int rc = check_cuda(cudaMemsetAsync(a.workspace, 0, kWsHeader, static_cast<cudaStream_t>(a.stream)),
                                "cudaMemsetAsync(decode scratch header)"))
            return rc;
    }
    const size_t rows = static_cast<size_t>(a.batch) * a.q_heads * splits;
    float* wsf = reinterpret_cast<float*>(static_cast<unsigned char*>(a.workspace) + kWsHeader);
    DecodeParams p{};
    p.q = static_cast<const __half*>(a.q);
    p.kc = static_cast<const __half*>(a.kc);
    p.kid = static_cast<const int8_t*>(a.kid);
    p.kp = a.kp, p.kb = a.km;
    p.vid = static_cast<const int8_t*>(a.vid);
    p.vp = a.vp, p.vb = a.vm;
    p.ks = static_cast<const __half*>(a.ks), p.vs = static_cast<const __half*>(a.vs);
    // the two wide arrays first: their rows stay 16-byte aligned for any row count
    p.ws_delta = wsf;
    p.ws_beta = wsf + rows * kHeadDim;
    p.ws_m = wsf + rows * (kHeadDim + kMaxClusters);
    p.ws_l = p.ws_m + rows;
    p.status = static_cast<uint32_t*>(a.workspace);
    p.inv_freq = a.inv_freq;
    p.tok_stride = a.tok_stride;
    p.kh = a.kv_heads, p.nh = a.q_heads, p.tokens = a.tokens, p.ck = a.ck, p.cv = a.cv;
    p.start_pos = a.start_pos, p.pos_q = a.pos_q, p.splits = splits, p.tiles_per_split = per;
    p.theta = a.theta, p.scaling = a.scaling;
    p.dyn = a.dyn;
    p.units = units, p.balanced = pp.balanced, p.grid = pp.grid;

    cudaStream_t s = static_cast<cudaStream_t>(a.stream);
    if (g_ev_start) cudaEventRecord(g_ev_start, s);
    int rc = gqa == 1 ? dispatch_layout<1>(p, layout, units, s)
             : gqa == 4 ? dispatch_layout<4>(p, layout, units, s)
                        : dispatch_layout<8>(p, layout, units, s);
    if (rc) return rc;
    if (g_ev_stop) cudaEventRecord(g_ev_stop, s);

    MergeParams mp{};
    mp.ws_m = p.ws_m, mp.ws_l = p.ws_l, mp.ws_delta = p.ws_delta, mp.ws_beta = p.ws_beta;
    mp.vc = static_cast<const __half*>(a.vc);
    mp.rq = static_cast<const __half*>(a.rq);
    mp.rk = static_cast<const __half*>(a.rk);
    mp.rv = static_cast<const __half*>(a.rv);
    mp.out = static_cast<__half*>(a.out);
    mp.out_m = a.out_m, mp.out_l = a.out_l;
    mp.kh = a.kv_heads, mp.nh = a.q_heads, mp.splits = splits, mp.cv = a.cv, mp.tr = a.recent_tokens;
    mp.scaling = a.scaling;
    mp.dyn = a.dyn, mp.recent_cap = a.dyn ? a.recent_cap : a.recent_tokens;
    mp.status = p.status;
    return launch_merge(mp, units, a.dyn ? a.recent_cap : a.recent_tokens, s);
}
}  // namespace

extern "C" int reskv_decode_bitmap_fp16(const void* q, const void* k_centroids, const void* k_ids,
                                        const void* k_payload, const void* k_bitmap, const void* v_centroids,
                                        const void* v_ids, const void* v_payload, const void* v_bitmap, int batch,
                                        int kv_heads, int q_heads, int tokens, int64_t tok_stride, int k_clusters,
                                        int v_clusters, int nnz, int start_pos, int pos_q, float rope_theta,
                                        const float* inv_freq, float scaling, int splits, const void* recent_q,
                                        const void* recent_k, const void* recent_v, int recent_tokens,
                                        void* workspace, size_t workspace_bytes_given, void* out, float* out_m,
                                        float* out_l, void* stream) {
    if (nnz != 32 && nnz != 64) return fail(RESKV_ERR_INVALID, "decode_bitmap_fp16: nnz must be 32 or 64, got %d", nnz);
    const DecodeArgs a{q, k_centroids, k_ids, k_payload, k_bitmap, nullptr, v_centroids, v_ids, v_payload, v_bitmap,
                       nullptr, batch, kv_heads, q_heads, tokens, tok_stride, k_clusters, v_clusters, start_pos, pos_q,
                       rope_theta, inv_freq, scaling, splits, recent_q, recent_k, recent_v, recent_tokens, workspace,
                       workspace_bytes_given, out, out_m, out_l, stream};
    return decode_common(a, nnz == 32 ? kBitmap32 : kBitmap64, true, false, "decode_bitmap_fp16");
}

extern "C" int reskv_decode_packed(int layout, int bits, const void* q, const void* k_centroids, const void* k_ids,
                                   const void* k_payload, const void* k_meta, const void* k_scale,
                                   const void* v_centroids, const void* v_ids, const void* v_payload,
                                   const void* v_meta, const void* v_scale, int batch, int kv_heads, int q_heads,
                                   int tokens, int64_t tok_stride, int k_clusters, int v_clusters, int start_pos,
                                   int pos_q, float rope_theta, const float* inv_freq, float scaling, int splits,
                                   const void* recent_q, const void* recent_k, const void* recent_v, int recent_tokens,
                                   void* workspace, size_t workspace_bytes_given, void* out, float* out_m,
                                   float* out_l, void* stream) {
    LayoutId id;
    bool meta = true, scale = false;
    if (layout == RESKV_LAYOUT_UNSTRUCTURED && (bits == 4 || bits == 2)) {
        id = bits == 4 ? kQuant4 : kQuant2, meta = false, scale = true;
    } else if (layout == RESKV_LAYOUT_TILED && bits == 16) {
        id = kTiled64;
    } else if (layout == RESKV_LAYOUT_STRUCTURED && bits == 16) {
        id = kStruct32;
    } else if (layout == RESKV_LAYOUT_STRUCTURED && bits == 4) {
        id = kStructInt4, scale = true;
    } else {
        return fail(RESKV_ERR_INVALID, "decode_packed: no kernel for layout %d with %d-bit residuals", layout, bits);
    }
    const DecodeArgs a{q, k_centroids, k_ids, k_payload, k_meta, k_scale, v_centroids, v_ids, v_payload, v_meta,
                       v_scale, batch, kv_heads, q_heads, tokens, tok_stride, k_clusters, v_clusters, start_pos, pos_q,
                       rope_theta, inv_freq, scaling, splits, recent_q, recent_k, recent_v, recent_tokens, workspace,
                       workspace_bytes_given, out, out_m, out_l, stream};
    return decode_common(a, id, meta, scale, "decode_packed");
}

extern "C" int reskv_decode_compact(int bits, int nnz, const void* q, const void* k_centroids, const void* k_ids,
                                    const void* k_payload, const void* k_bitmap, const void* k_scale,
                                    const void* v_centroids, const void* v_ids, const void* v_payload,
                                    const void* v_bitmap, const void* v_scale, int batch, int kv_heads, int q_heads,
                                    int tokens, int64_t tok_stride, int k_clusters, int v_clusters, int start_pos,
                                    int pos_q, float rope_theta, const float* inv_freq, float scaling, int splits,
                                    const void* recent_q, const void* recent_k, const void* recent_v, int recent_tokens,
                                    void* workspace, size_t workspace_bytes_given, void* out, float* out_m,
                                    float* out_l, void* stream) {
    LayoutId id;
    if (bits == 4 && nnz == 64) {
        id = kCompact4x64;
    } else if (bits == 4 && nnz == 32) {
        id = kCompact4x32;
    } else if (bits == 2 && nnz == 64) {
        id = kCompact2x64;
    } else {
        return fail(RESKV_ERR_INVALID, "decode_compact: no kernel for %d retained %d-bit codes per token", nnz, bits);
    }
    const DecodeArgs a{q, k_centroids, k_ids, k_payload, k_bitmap, k_scale, v_centroids, v_ids, v_payload, v_bitmap,
                       v_scale, batch, kv_heads, q_heads, tokens, tok_stride, k_clusters, v_clusters, start_pos, pos_q,
                       rope_theta, inv_freq, scaling, splits, recent_q, recent_k, recent_v, recent_tokens, workspace,
                       workspace_bytes_given, out, out_m, out_l, stream};
    return decode_common(a, id, true, true, "decode_compact");
}

extern "C" int reskv_decode_step(int layout, int bits, int nnz, const void* q, const void* k_centroids,
                                 const void* k_ids, const void* k_payload, const void* k_meta, const void* k_scale,
                                 const void* v_centroids, const void* v_ids, const void* v_payload,
                                 const void* v_meta, const void* v_scale, int batch, int kv_heads, int q_heads,
                                 int tokens, int64_t tok_stride, int k_clusters, int v_clusters, int start_pos,
                                 float rope_theta, const float* inv_freq, float scaling, int splits,
                                 const void* recent_q, const void* window_k, const void* window_v,
                                 int window_capacity, const int32_t* step_state, void* workspace,
                                 size_t workspace_bytes_given, void* out, void* stream) {
    if (!step_state) return fail(RESKV_ERR_INVALID, "decode_step: null step state");
    LayoutId id;
    bool meta = true, scale = false;
    if (layout == RESKV_LAYOUT_UNSTRUCTURED && bits == 16 && (nnz == 32 || nnz == 64)) {
        id = nnz == 32 ? kBitmap32 : kBitmap64;
    } else if (layout == RESKV_LAYOUT_UNSTRUCTURED && (bits == 4 || bits == 2)) {
        id = bits == 4 ? kQuant4 : kQuant2, meta = false, scale = true;
    } else if (layout == RESKV_LAYOUT_TILED && bits == 16) {
        id = kTiled64;
    } else if (layout == RESKV_LAYOUT_STRUCTURED && bits == 16) {
        id = kStruct32;
    } else if (layout == RESKV_LAYOUT_STRUCTURED && bits == 4) {
        id = kStructInt4, scale = true;
    } else if (layout == RESKV_LAYOUT_COMPACT && bits == 4 && (nnz == 64 || nnz == 32)) {
        id = nnz == 64 ? kCompact4x64 : kCompact4x32, scale = true;
    } else if (layout == RESKV_LAYOUT_COMPACT && bits == 2 && nnz == 64) {
        id = kCompact2x64, scale = true;
    } else {
        return fail(RESKV_ERR_INVALID, "decode_step: no kernel for layout %d with %d-bit residuals (nnz %d)", layout, bits, nnz);
    }
    DecodeArgs a{q, k_centroids, k_ids, k_payload, k_meta, k_scale, v_centroids, v_ids, v_payload, v_meta, v_scale,
                 batch, kv_heads, q_heads, tokens, tok_stride, k_clusters, v_clusters, start_pos, 0, rope_theta,
                 inv_freq, scaling, splits, recent_q, window_k, window_v, 0, workspace, workspace_bytes_given, out,
                 nullptr, nullptr, stream};
    a.dyn = step_state;
    a.recent_cap = window_capacity;
    return decode_common(a, id, meta, scale, "decode_step");
}

// ---- decode without any caller- or library-side allocation -----------------------------
// Scratch for the split partials lives in this fixed array inside the library image.
// Every GPU that loads the library carries it until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[RESKV_NOALLOC_SCRATCH_BYTES];

namespace {
// Device address of g_noalloc_scratch on the current device.  In host code the
// array's name is only a handle for the runtime, not something a kernel can
// dereference, so the address is looked up once per device (with that device
// current) and remembered.  The remembered value is written without a lock: two
// host threads that make their first call on a device together both look the
// address up and store the same value.
int noalloc_scratch_address(void** out) {
    static void* cached[64] = {nullptr};
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    if (dev < 0 || dev >= 64) return fail(RESKV_ERR_LIMIT, "decode_bitmap_fp16_noalloc: device index %d not supported", dev);
    if (!cached[dev]) {
        void* ptr = nullptr;
        if (int rc = check_cuda(cudaGetSymbolAddress(&ptr, g_noalloc_scratch),
                                "cudaGetSymbolAddress(built-in decode scratch)"))
            return rc;
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return RESKV_OK;
}
}  // namespace

extern "C" int reskv_decode_bitmap_fp16_noalloc(const void* q, const void* k_centroids, const void* k_ids,
                                                const void* k_payload, const void* k_bitmap,
                                                const void* v_centroids, const void* v_ids, const void* v_payload,
                                                const void* v_bitmap, int batch, int kv_heads, int q_heads,
                                                int tokens, int64_t tok_stride, int k_clusters, int v_clusters,
                                                int nnz, int start_pos, int pos_q, float rope_theta,
                                                const float* inv_freq, float scaling, int splits,
                                                const void* recent_q, const void* recent_k, const void* recent_v,
                                                int recent_tokens, void* out, float* out_m, float* out_l,
                                                void* stream) {
    if (batch < 1 || kv_heads < 1 || q_heads < 1 || tokens < 1)
        return fail(RESKV_ERR_INVALID, "decode_bitmap_fp16_noalloc: batch, heads and tokens must be positive");
    if (nnz != 32 && nnz != 64)
        return fail(RESKV_ERR_INVALID, "decode_bitmap_fp16_noalloc: nnz must be 32 or 64, got %d", nnz);
    // the same partial plan as the allocating entry point, to size the scratch first
    const int eff = plan_partials(batch * kv_heads, tokens, splits, g_variant == 0, false, tok_stride).slots;
    const size_t need = workspace_bytes(batch * q_heads, eff);
    if (need > static_cast<size_t>(RESKV_NOALLOC_SCRATCH_BYTES))
        return fail(RESKV_ERR_LIMIT,
                    "decode_bitmap_fp16_noalloc: %d query heads x %d splits need %zu bytes of scratch, the built-in "
                    "array holds %d; pass fewer splits or call reskv_decode_bitmap_fp16 with your own workspace",
                    batch * q_heads, eff, need, RESKV_NOALLOC_SCRATCH_BYTES);
    void* scratch = nullptr;
    if (int rc = noalloc_scratch_address(&scratch)) return rc;
    // the array still holds the previous call's data; only the status header has to start at zero (every
    // partial slot that the merge reads is written or marked empty by this call's partial kernel first):
    // decode_common clears it once the arguments have been accepted
    DecodeArgs a{q, k_centroids, k_ids, k_payload, k_bitmap, nullptr, v_centroids, v_ids, v_payload, v_bitmap,
                 nullptr, batch, kv_heads, q_heads, tokens, tok_stride, k_clusters, v_clusters, start_pos, pos_q,
                 rope_theta, inv_freq, scaling, splits, recent_q, recent_k, recent_v, recent_tokens, scratch,
                 static_cast<size_t>(RESKV_NOALLOC_SCRATCH_BYTES), out, out_m, out_l, stream};
    a.clear_status = true;
    return decode_common(a, nnz == 32 ? kBitmap32 : kBitmap64, true, false, "decode_bitmap_fp16_noalloc");
}

extern "C" int reskv_decode_noalloc_status(uint32_t* status_out, void* stream) {
    if (!status_out) return fail(RESKV_ERR_INVALID, "decode_noalloc_status: null destination");
    void* scratch = nullptr;
    if (int rc = noalloc_scratch_address(&scratch)) return rc;
    return check_cuda(cudaMemcpyAsync(status_out, scratch, sizeof(uint32_t), cudaMemcpyDeviceToHost,
                                      static_cast<cudaStream_t>(stream)),
                      "cudaMemcpyAsync(built-in decode scratch status)");
}

static int merge_recent_common(const void* comp_out, const float* comp_m, const float* comp_l, const float* scores,
                               const void* rq, const void* rk, const void* rv, int batch, int kv_heads, int q_heads,
                               int recent_tokens, float scaling, void* merged, void* stream, const char* who) {
    if (!comp_out || !comp_m || !comp_l || !rv || !merged) return fail(RESKV_ERR_INVALID, "%s: null tensor pointer", who);
    if (batch < 1 || kv_heads < 1 || q_heads < 1 || q_heads % kv_heads)
        return fail(RESKV_ERR_INVALID, "%s: bad batch or head counts", who);
    if (recent_tokens < 1) return fail(RESKV_ERR_INVALID, "%s: recent_tokens must be positive", who);
    if (recent_tokens > kMaxRecent)
        return fail(RESKV_ERR_LIMIT, "%s: at most %d recent tokens, got %d", who, kMaxRecent, recent_tokens);
    if ((rk && !aligned16(rk)) || !aligned16(rv))
        return fail(RESKV_ERR_INVALID, "%s: recent keys and values must be 16-byte aligned", who);
    MergeParams mp{};
    mp.ws_m = comp_m, mp.ws_l = comp_l;
    mp.comp_out = static_cast<const __half*>(comp_out);
    mp.rscores = scores;
    mp.rq = static_cast<const __half*>(rq);
    mp.rk = static_cast<const __half*>(rk);
    mp.rv = static_cast<const __half*>(rv);
    mp.out = static_cast<__half*>(merged);
    mp.kh = kv_heads, mp.nh = q_heads, mp.splits = 0, mp.tr = recent_tokens, mp.scaling = scaling;
    mp.recent_cap = recent_tokens;
    return launch_merge(mp, batch * kv_heads, recent_tokens, static_cast<cudaStream_t>(stream));
}

extern "C" int reskv_merge_recent_scores(const void* comp_out, const float* comp_m, const float* comp_l,
                                         const float* scores, const void* recent_v, int batch, int kv_heads,
                                         int q_heads, int recent_tokens, void* merged, void* stream) {
    if (!scores) return fail(RESKV_ERR_INVALID, "merge_recent_scores: null scores");
    return merge_recent_common(comp_out, comp_m, comp_l, scores, nullptr, nullptr, recent_v, batch, kv_heads, q_heads,
                               recent_tokens, 1.f, merged, stream, "merge_recent_scores");
}

extern "C" int reskv_merge_recent_qk(const void* comp_out, const float* comp_m, const float* comp_l,
                                     const void* recent_q, const void* recent_k, const void* recent_v, int batch,
                                     int kv_heads, int q_heads, int recent_tokens, float scaling, void* merged,
                                     void* stream) {
    if (!recent_q || !recent_k) return fail(RESKV_ERR_INVALID, "merge_recent_qk: null rotated q or k");
    return merge_recent_common(comp_out, comp_m, comp_l, nullptr, recent_q, recent_k, recent_v, batch, kv_heads,
                               q_heads, recent_tokens, scaling, merged, stream, "merge_recent_qk");
}

// Tensor-core version of the partial decode kernel, generic over the residual layout
// (the description below is written for the unstructured FP16 bitmap layout; the
// other layouts only differ in how a lane obtains the 16 coordinates of a field,
// see the *Field structs).  Included by decode_bitmap.cu and decode_packed_mma.cu
// (needs DecodeParams and rope_freq from decode_common.cuh).
//
// Why: the warp-per-token kernel spends ~250 warp instructions per (token, KV head)
// and is issue bound at 8 % of HBM bandwidth.  Here a warp handles blocks of 16
// tokens and both contractions run on mma.sync.m16n8k16 tiles:
//
//   S[16 tok x 8 heads]   = K'[16 tok x 128] . Qt^T          (8 k-steps, Qt split hi+lo FP16)
//   O^T[128 x 8 heads]   += Vres^T[128 x 16 tok] . P[16 tok x 8 heads]   (8 m-blocks)
//
// The contraction order of an MMA is free, so coordinates are assigned to
// fragment slots such that every lane owns *contiguous* 16-coordinate fields of
// a token: lane (g = lane / 4, q = lane % 4) builds, for K, tokens g and g + 8,
// coordinates [16q, 16q+16) and their RoPE partners [64+16q, 64+16q+16); for V,
// tokens {2q, 2q+1, 2q+8, 2q+9}, coordinates [16g, 16g+16).  A field is one
// 16-bit slice of the token's bitmap; its retained values are consecutive in the
// payload, so decoding is a walk "bit set ? *ptr++ : 0" with no popcount per
// coordinate (one table of 8 rank bases per token is built per block).
//
// RoPE: a token at tile offset j of a tile starting at position P0 scores
//   < R(pos_q) q, R(P0 + j) k >  =  < R(pos_q - P0) q, R(j) k > ,
// so keys are rotated by the in-tile offset only -- sin/cos of j * f_i come from a
// 64 x 64 shared-memory table built once per CTA -- and the query is re-rotated
// once per 64-token tile (by all threads, incrementally) into MMA B-fragment
// order.  Softmax keeps a lazily updated running maximum per head (rescale only
// when it grows by more than 2^8), P is rounded to FP16 once and that rounded
// value is used for the sum, the cluster masses and the PV product alike.  The
// cluster masses beta[value cluster][head] are a third contraction on the same P,
// onehot(value id)^T . P (one-hot rows from a packed FP16 compare of the ids), and
// the PV MMAs follow the value walks two coordinates at a time.
//
// Staging: metadata by one bulk copy per tile, payload rows of the sparse FP16
// layouts by 16-byte cp.async pieces of all threads into rows padded by 16 bytes
// (lanes that walk the same field of different tokens then start in different
// banks); one mbarrier per ring slot counts both, every wait on it is bounded.
//
// Precision: a single FP16 rounding of the rotated key is not enough (outlier
// channels put the score error at ~1e-3, ten times the output tolerance on short
// contexts), so K' enters the MMA as hi + lo FP16 halves: S = K'hi.Qhi + K'hi.Qlo
// + K'lo.Qhi.  The sm_100 mixed-precision instructions keep that cheap:
// add.f32.f16 adds the FP16 residual to the FP32 centroid in one instruction and
// fma.f32.f16 forms lo = k' - hi without unpacking.
#pragma once

namespace mma {

constexpr int kTileM = 64;        // tokens per pipeline stage
constexpr int kWarpsM = 4;        // one 16-token block per warp and tile
constexpr int kThreadsM = kWarpsM * 32;
constexpr int kCenStride = 132;   // floats per centroid row in shared memory (row r starts 4r banks on)
constexpr int kTrigStride = 64;   // float2 per row of the sin/cos table (swizzled, see trig_index)
constexpr int kQStride = 132;     // halfs per query row
constexpr int kQSets = 2;         // query stored as FP16 hi and lo
constexpr float kRescaleThreshold = 8.0f;  // log2 units

// Payload rows are staged kPad bytes apart from dense when the layout asks for it: lanes that walk
// the same field of different tokens then start in different banks.
template <class ML>
struct StageM {
    alignas(16) unsigned char kp[kTileM * (ML::kPayloadBytes + ML::kPad)];
    alignas(16) unsigned char vp[kTileM * (ML::kPayloadBytes + ML::kPad)];
    alignas(16) unsigned char km[kTileM * (ML::kMetaBytes ? ML::kMetaBytes : 1)];
    alignas(16) unsigned char vm[kTileM * (ML::kMetaBytes ? ML::kMetaBytes : 1)];
};

template <class ML>
constexpr int stages_for() {
    return sizeof(StageM<ML>) <= 12800 ? 3 : 2;
}

// The sin/cos values a lane keeps in registers are read once from a shared table (64 tile offsets x 64
// frequencies, 32 KB) that aliases the ring of stages.
template <class ML>
constexpr int trig_rows() {
    return kTileM;
}

// Shared-memory layouts chosen so that the 16-byte loads of a quarter warp
// (lanes g = 2k, 2k+1; q = 0..3) fall into distinct banks.
//
// sin/cos table: row j (tile offset), frequency i = 16q + 4ks + 2e + u.  The four
// lanes q of one (ks, e) read neighbouring 16-byte units; odd rows swap the two
// 64-byte halves of every 128-byte line.
__device__ __forceinline__ int trig_index(int j, int i) {
    const int q = i >> 4, ks = (i >> 2) & 3, e = (i >> 1) & 1, u = i & 1;
    const int unit = (((ks * 2 + e) * 4 + q) ^ ((j & 1) << 2));
    return j * kTrigStride + unit * 2 + u;
}
// centroid row (FP32): coordinate d -> field f = d / 16, 16-byte unit (d / 4) % 4,
// units of fields 2, 3, 6, 7 are swapped pairwise so lanes q and q + 2 differ.
__device__ __forceinline__ int cen_index(int d) {
    const int f = d >> 4, unit = ((d >> 2) & 3) ^ ((f >> 1) & 1);
    return f * 16 + unit * 4 + (d & 3);
}

// d = fp16(bits) + c, one instruction (sm_100 mixed-precision add)
__device__ __forceinline__ float add_f16_f32(unsigned short bits, float c) {
    float d;
    asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"(bits), "f"(c));
    return d;
}
// d = fp16(a) * fp16(b) + c
__device__ __forceinline__ float fma_f16_f16_f32(unsigned short a, unsigned short b, float c) {
    float d;
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
    return d;
}
// (hi, lo) FP16 pairs of two FP32 values: hi = fp16(x), lo = fp16(x - hi)
__device__ __forceinline__ void split_h2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(x0, x1);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    const unsigned short minus_one = 0xbc00;
    const float l0 = fma_f16_f16_f32(__half_as_ushort(__low2half(h)), minus_one, x0);
    const float l1 = fma_f16_f16_f32(__half_as_ushort(__high2half(h)), minus_one, x1);
    const __half2 l = __floats2half2_rn(l0, l1);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

// The sin/cos table is only read once per CTA (into registers, before the first tile is requested), so it
// shares its memory with the ring of stages.
template <class ML>
constexpr size_t stage_region_bytes() {
    constexpr size_t ring = sizeof(StageM<ML>) * stages_for<ML>();
    constexpr size_t table = trig_rows<ML>() * kTrigStride * sizeof(float2);
    return ring > table ? ring : table;
}

template <int GQA, class ML>
constexpr size_t smem_bytes(int ck) {
    return stage_region_bytes<ML>() +
           static_cast<size_t>(ck) * kCenStride * sizeof(float) + 2 * kQSets * GQA * kQStride * sizeof(__half) +
           kWarpsM * 2 * 16 * sizeof(uint2) + kWarpsM * GQA * kMaxClusters * sizeof(float);
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Byte offset, inside a token's 16-byte bitmap, of the 16-bit field that covers
// coordinates [16f, 16f+16) (bit 15 = first coordinate).
__device__ __forceinline__ int field_offset(int f) { return ((f & 4) ? 8 : 0) + 6 - 2 * (f & 3); }

// Number of retained coordinates before each of the eight fields, one byte each.
__device__ __forceinline__ uint2 rank_bases(const uint4 bm) {
    const uint32_t w0 = bm.y, w1 = bm.x, w2 = bm.w, w3 = bm.z;
    const uint32_t r1 = __popc(w0 >> 16), r2 = __popc(w0);
    const uint32_t r3 = r2 + __popc(w1 >> 16), r4 = r2 + __popc(w1);
    const uint32_t r5 = r4 + __popc(w2 >> 16), r6 = r4 + __popc(w2);
    const uint32_t r7 = r6 + __popc(w3 >> 16);
    return make_uint2((r1 << 8) | (r2 << 16) | (r3 << 24), r4 | (r5 << 8) | (r6 << 16) | (r7 << 24));
}

// One step of a field walk: the next coordinate's raw FP16 bits, or 0.
__device__ __forceinline__ uint32_t walk16(uint32_t field, int e, const __half*& ptr) {
    uint32_t v = 0;
    if (field & (0x8000u >> e)) {
        v = *reinterpret_cast<const unsigned short*>(ptr);
        ++ptr;
    }
    return v;
}

__device__ __forceinline__ float h2f_bits(uint32_t bits) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits)));
}

// ---- fields: the 16 coordinates [16 f, 16 f + 16) of one token, as a lane consumes them --------
// add4(ks, k, scale): k[e] += residual of coordinate 4 ks + e   (key side; k holds the FP32 centroid)
// bits4(ks, h):       h[e]  = FP16 bit pattern of the coordinate's MMA operand value (value side)
// Both must be called with ks = 0, 1, 2, 3 in order (the sparse layouts walk a pointer).

// Sparse FP16 layouts: a 16-bit keep mask (bit 15 = first coordinate) and a pointer to the
// field's first retained value; retained values are consecutive in the payload row.
struct WalkField {
    static constexpr bool kSlotwise = true;  // offers add1 / bits1: callers interleave the walks of several fields
    uint32_t mask;
    const __half* ptr;
    __device__ __forceinline__ void add1(int slot, float& k) {
        if (mask & (0x8000u >> slot)) {
            k = add_f16_f32(*reinterpret_cast<const unsigned short*>(ptr), k);
            ++ptr;
        }
    }
    __device__ __forceinline__ uint32_t bits1(int slot) { return walk16(mask, slot, ptr); }
    __device__ __forceinline__ void add4(int ks, float (&k)[4], unsigned short) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (mask & (0x8000u >> (4 * ks + e))) {
                k[e] = add_f16_f32(*reinterpret_cast<const unsigned short*>(ptr), k[e]);
                ++ptr;
            }
        }
    }
    __device__ __forceinline__ void bits4(int ks, uint32_t (&h)[4]) {
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = walk16(mask, 4 * ks + e, ptr);
    }
};

// Unstructured FP16: MSB-first bitmap; rank bases from the per-block table `pre` (8 bytes per token).
template <int NNZ>
struct LayoutMmaBitmap {
    static constexpr int kPayloadBytes = NNZ * 2, kMetaBytes = 16, kPad = 16;
    static constexpr bool kScale = false, kPrefix = true, kScaleP = false;
    using Field = WalkField;
    __device__ static __forceinline__ Field field(const unsigned char* pay, const unsigned char* meta,
                                                  const unsigned char* pre, int tok, int f, bool ok) {
        Field fd;
        fd.mask = ok ? *reinterpret_cast<const unsigned short*>(meta + tok * 16 + field_offset(f)) : 0u;
        fd.ptr = reinterpret_cast<const __half*>(pay + tok * (kPayloadBytes + kPad)) + pre[(tok & 15) * 8 + f];
        return fd;
    }
};

// Tiled FP16 (INDEXED = false): one LSB-first 16-bit mask per tile = field.  Structured 4:16
// (INDEXED = true): four 4-bit in-tile indices.  Metadata word w carries tile 2w (low half) and
// 2w + 1 (high half), i.e. tile f sits at byte 2 f; its values start at f * NNZ / 8.
template <int NNZ, bool INDEXED>
struct LayoutMmaTiled {
    static constexpr int kPayloadBytes = NNZ * 2, kMetaBytes = 16, kPad = 16;
    static constexpr bool kScale = false, kPrefix = false, kScaleP = false;
    using Field = WalkField;
    __device__ static __forceinline__ Field field(const unsigned char* pay, const unsigned char* meta,
                                                  const unsigned char*, int tok, int f, bool ok) {
        const uint32_t code = ok ? *reinterpret_cast<const unsigned short*>(meta + tok * 16 + 2 * f) : 0u;
        Field fd;
        if constexpr (INDEXED) {
            // four in-tile indices -> keep mask with bit 15 = first coordinate
            const uint32_t c = code;
            fd.mask = ok ? ((0x8000u >> (c & 15u)) | (0x8000u >> ((c >> 4) & 15u)) | (0x8000u >> ((c >> 8) & 15u)) |
                            (0x8000u >> (c >> 12)))
                         : 0u;
        } else {
            fd.mask = __brev(code) >> 16;  // LSB-first -> bit 15 = first coordinate
        }
        fd.ptr = reinterpret_cast<const __half*>(pay + tok * (kPayloadBytes + kPad)) + f * (NNZ / 8);
        return fd;
    }
};

// Pair of small integer codes -> two exact FP16 integers.  `x` holds code a in bits [0, BITS) and
// code b in bits [16 + SHIFT, 16 + SHIFT + BITS) (both as stored, two's complement).  Setting the
// FP16 exponent bits makes each half 1024 + (code ^ sign) * 2^shift; one HFMA2 rescales and removes
// the offsets.
template <int BITS, int SHIFT>
__device__ __forceinline__ uint32_t codes_to_h2(uint32_t x) {
    constexpr uint32_t kSign = 1u << (BITS - 1);
    constexpr uint32_t kKeep = ((1u << BITS) - 1u) | (((1u << BITS) - 1u) << (16 + SHIFT));
    const uint32_t y = ((x & kKeep) ^ (kSign | (kSign << (16 + SHIFT)))) | 0x64006400u;
    const __half2 mul = __floats2half2_rn(1.0f, 1.0f / static_cast<float>(1 << SHIFT));
    const __half2 sub = __floats2half2_rn(-1024.0f - static_cast<float>(kSign),
                                          -(1024.0f / static_cast<float>(1 << SHIFT)) - static_cast<float>(kSign));
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&y), mul, sub);
    return *reinterpret_cast<const uint32_t*>(&r);
}

// Unstructured INT4 / INT2: all 16 coordinates of a field are stored (2 words / 1 word);
// residual = code * scale (scale FP16 per token).
template <int BITS>
struct QuantField {
    static constexpr bool kSlotwise = false;
    uint32_t w0, w1;
    // codes of coordinates 4 ks + {0,1} and 4 ks + {2,3} as FP16 pairs
    __device__ __forceinline__ void pairs(int ks, uint32_t& p01, uint32_t& p23) const {
        if constexpr (BITS == 4) {
            const uint32_t w = (ks < 2) ? w0 : w1;
            const uint32_t two = (w >> (16 * (ks & 1))) & 0xffffu;      // coordinates 4ks..4ks+3, a nibble each
            const uint32_t b0 = two & 0xffu, b1 = two >> 8;
            p01 = codes_to_h2<4, 4>(b0 | (b0 << 16));                    // lo nibble -> low half, hi nibble (x16) -> high half
            p23 = codes_to_h2<4, 4>(b1 | (b1 << 16));
        } else {
            const uint32_t byte = (w0 >> (8 * ks)) & 0xffu;              // four 2-bit codes
            const uint32_t n0 = byte & 15u, n1 = byte >> 4;
            p01 = codes_to_h2<2, 2>(n0 | (n0 << 16));
            p23 = codes_to_h2<2, 2>(n1 | (n1 << 16));
        }
    }
    __device__ __forceinline__ void add4(int ks, float (&k)[4], unsigned short scale) const {
        uint32_t p01, p23;
        pairs(ks, p01, p23);
        k[0] = fma_f16_f16_f32(static_cast<unsigned short>(p01 & 0xffffu), scale, k[0]);
        k[1] = fma_f16_f16_f32(static_cast<unsigned short>(p01 >> 16), scale, k[1]);
        k[2] = fma_f16_f16_f32(static_cast<unsigned short>(p23 & 0xffffu), scale, k[2]);
        k[3] = fma_f16_f16_f32(static_cast<unsigned short>(p23 >> 16), scale, k[3]);
    }
    __device__ __forceinline__ void bits4(int ks, uint32_t (&h)[4]) const {
        uint32_t p01, p23;
        pairs(ks, p01, p23);
        h[0] = p01 & 0xffffu, h[1] = p01 >> 16, h[2] = p23 & 0xffffu, h[3] = p23 >> 16;
    }
};

template <int BITS>
struct LayoutMmaQuant {
    static constexpr int kPayloadBytes = 16 * BITS, kMetaBytes = 0, kPad = 0;
    static constexpr bool kScale = true, kPrefix = false, kScaleP = true;
    using Field = QuantField<BITS>;
    __device__ static __forceinline__ Field field(const unsigned char* pay, const unsigned char*,
                                                  const unsigned char*, int tok, int f, bool ok) {
        Field fd{0u, 0u};
        if (ok) {
            if constexpr (BITS == 4) {
                const uint2 w = *reinterpret_cast<const uint2*>(pay + tok * 64 + 8 * f);
                fd.w0 = w.x, fd.w1 = w.y;
            } else {
                fd.w0 = *reinterpret_cast<const uint32_t*>(pay + tok * 32 + 4 * f);
            }
        }
        return fd;
    }
};

// Compact quantised layout: a 16-bit keep mask like the FP16 bitmap layout, but the field's retained
// coordinates are BITS-wide codes inside the token's packed row.  At most 16 codes of 4 bits: the
// field's codes fit one 64-bit window, fetched once (three aligned words, funnel-shifted to the
// field's first code) and consumed from the low end.  A code enters arithmetic as the FP16 number
// 1024 + (code ^ sign), i.e. bits 0x6400 | (code ^ sign); the offset 1024 + sign is removed by the
// consumer (key side: folded into the FP32 accumulator start; value side: one HADD2 per pair).
template <int BITS>
struct CompactField {
    static constexpr bool kSlotwise = false;
    static constexpr uint32_t kSign = 1u << (BITS - 1);
    static constexpr uint32_t kZero = 0x6400u | kSign;  // FP16 bits of the value that stands for code 0
    uint32_t mask, lo, hi;
    __device__ __forceinline__ uint32_t next() {  // FP16 bits of the next retained code; advances the window
        const uint32_t h = ((lo & ((1u << BITS) - 1u)) ^ kZero);
        lo = __funnelshift_r(lo, hi, BITS);
        hi >>= BITS;
        return h;
    }
    __device__ __forceinline__ void add4(int ks, float (&k)[4], unsigned short scale) {
        // k += code * scale for retained coordinates (code = h - (1024 + sign), exact in FP16)
        const __half off = __float2half_rn(1024.f + static_cast<float>(kSign));
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (mask & (0x8000u >> (4 * ks + e))) {
                const __half code = __hsub(__ushort_as_half(static_cast<unsigned short>(next())), off);
                k[e] = fma_f16_f16_f32(__half_as_ushort(code), scale, k[e]);
            }
        }
    }
    __device__ __forceinline__ void bits4(int ks, uint32_t (&h)[4]) {
        uint32_t raw[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) raw[e] = (mask & (0x8000u >> (4 * ks + e))) ? next() : kZero;
        // remove the offset exactly: values are integers in [-8, 7]
        const __half2 off = __float2half2_rn(-(1024.f + static_cast<float>(kSign)));
        const uint32_t p01 = raw[0] | (raw[1] << 16), p23 = raw[2] | (raw[3] << 16);
        const __half2 r01 = __hadd2(*reinterpret_cast<const __half2*>(&p01), off);
        const __half2 r23 = __hadd2(*reinterpret_cast<const __half2*>(&p23), off);
        const uint32_t q01 = *reinterpret_cast<const uint32_t*>(&r01), q23 = *reinterpret_cast<const uint32_t*>(&r23);
        h[0] = q01 & 0xffffu, h[1] = q01 >> 16, h[2] = q23 & 0xffffu, h[3] = q23 >> 16;
    }
};

template <int BITS, int NNZ>
struct LayoutMmaCompact {
    static constexpr int kPayloadBytes = NNZ * BITS / 8, kMetaBytes = 16, kPad = 0;
    static constexpr bool kScale = true, kPrefix = true, kScaleP = true;
    static_assert(kPayloadBytes % 16 == 0, "packed rows must be whole 16-byte pieces");
    using Field = CompactField<BITS>;
    __device__ static __forceinline__ Field field(const unsigned char* pay, const unsigned char* meta,
                                                  const unsigned char* pre, int tok, int f, bool ok) {
        Field fd;
        fd.mask = ok ? *reinterpret_cast<const unsigned short*>(meta + tok * 16 + field_offset(f)) : 0u;
        // first code of the field = rank base * BITS bits into the row; words past the row's end are
        // never consumed (a field holds at most popcount(mask) codes), so their index is clamped
        constexpr int kWords = kPayloadBytes / 4;
        const uint32_t* row = reinterpret_cast<const uint32_t*>(pay + tok * kPayloadBytes);
        const int bit = pre[(tok & 15) * 8 + f] * BITS, w = bit >> 5, sh = bit & 31;
        const uint32_t w0 = row[min(w, kWords - 1)], w1 = row[min(w + 1, kWords - 1)], w2 = row[min(w + 2, kWords - 1)];
        fd.lo = __funnelshift_r(w0, w1, sh);
        fd.hi = __funnelshift_r(w1, w2, sh);
        return fd;
    }
};

// 1-of-4 structured INT4: per 4-coordinate group one signed nibble and a 2-bit position.
struct StructInt4Field {
    static constexpr bool kSlotwise = false;
    uint32_t c01, c23;  // the field's four group codes as FP16 pairs
    uint32_t sel;       // four 2-bit in-group positions
    __device__ __forceinline__ unsigned short code(int ks) const {
        const uint32_t p = (ks < 2) ? c01 : c23;
        return static_cast<unsigned short>((ks & 1) ? (p >> 16) : (p & 0xffffu));
    }
    __device__ __forceinline__ void add4(int ks, float (&k)[4], unsigned short scale) const {
        const uint32_t pos = (sel >> (2 * ks)) & 3u;
        const unsigned short c = code(ks);
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (pos == static_cast<uint32_t>(e)) k[e] = fma_f16_f16_f32(c, scale, k[e]);
    }
    __device__ __forceinline__ void bits4(int ks, uint32_t (&h)[4]) const {
        const uint32_t pos = (sel >> (2 * ks)) & 3u;
        const uint32_t c = code(ks);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = (pos == static_cast<uint32_t>(e)) ? c : 0u;
    }
};

struct LayoutMmaStructInt4 {
    static constexpr int kPayloadBytes = 16, kMetaBytes = 8, kPad = 0;
    static constexpr bool kScale = true, kPrefix = false, kScaleP = true;
    using Field = StructInt4Field;
    __device__ static __forceinline__ Field field(const unsigned char* pay, const unsigned char* meta,
                                                  const unsigned char*, int tok, int f, bool ok) {
        Field fd{0u, 0u, 0u};
        if (ok) {
            // groups 4f..4f+3: nibbles = 16 bits at byte 2f of the packed row, positions = byte f of the metadata row
            const uint32_t nib = *reinterpret_cast<const unsigned short*>(pay + tok * 16 + 2 * f);
            const uint32_t b0 = nib & 0xffu, b1 = nib >> 8;
            fd.c01 = codes_to_h2<4, 4>(b0 | (b0 << 16));
            fd.c23 = codes_to_h2<4, 4>(b1 | (b1 << 16));
            fd.sel = meta[tok * 8 + f];
        }
        return fd;
    }
};

#ifndef RESKV_MMA_CTAS_PER_SM
#define RESKV_MMA_CTAS_PER_SM 2  // resident CTAs the register allocation aims at (4 warps each)
#endif

// BETA = 16-cluster blocks of the cluster-mass accumulators: 4 serves every value-centroid count, 2 (counts up to
// 32, eight registers fewer) is 2 % faster and is what the launchers pick while the table is that small.
template <int GQA, class ML, int BETA = 4>
__global__ void __launch_bounds__(kThreadsM, RESKV_MMA_CTAS_PER_SM) decode_mma_kernel(const DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int kStages = stages_for<ML>();
    constexpr int kItems = (GQA * 32 + kThreadsM - 1) / kThreadsM;  // query items per thread
    // With four query heads the eight columns of the score MMA hold the query's FP16 hi halves (columns
    // 0..3) next to its lo halves (columns 4..7): one MMA per key half instead of two, the two columns of
    // a head are added afterwards (lanes q and q ^ 2).
    constexpr bool kPackQ = GQA == 4;
    using StageT = StageM<ML>;
    using Field = typename ML::Field;
    StageT* stages = reinterpret_cast<StageT*>(smem_raw);
    float2* trig = reinterpret_cast<float2*>(smem_raw);  // aliases the stages: dead before the first copy is issued
    float* kc_s = reinterpret_cast<float*>(smem_raw + stage_region_bytes<ML>());
    __half* qf = reinterpret_cast<__half*>(kc_s + static_cast<size_t>(p.ck) * kCenStride);  // [2 bufs][hi, lo][GQA][kQStride]
    uint2* pre = reinterpret_cast<uint2*>(qf + 2 * kQSets * GQA * kQStride);  // [warps][K, V][16]
    float* beta_s = reinterpret_cast<float*>(pre + kWarpsM * 2 * 16);  // [warps][GQA][64]
    __shared__ uint64_t full_bar[kStages];
    __shared__ float red_m[GQA][kWarpsM];
    __shared__ float red_l[GQA][kWarpsM];
    __shared__ uint32_t timed_out;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, qd = lane & 3;
    const int tokens = token_count(p);
    const int total_tiles = (tokens + kTileM - 1) / kTileM;
    // Work of the launch = the tiles of all units laid end to end, every unit padded to n_pad tiles.  CTA c
    // takes the range [c * chunk, (c + 1) * chunk) and walks it unit by unit; the part of one unit inside
    // the range is a *segment* and produces one partial result (slot = number of CTAs that started earlier
    // on the same unit).  Balanced schedule: n_pad = tiles of a unit and chunk = all tiles / CTAs, so every
    // CTA streams the same number of tiles and sets its tables up once; fixed-split schedule: chunk = tiles
    // per split and n_pad = chunk * splits, i.e. exactly one segment per CTA.
    int n_pad, chunk;
    if (p.balanced) {
        n_pad = max(total_tiles, 1);
        chunk = p.dyn ? static_cast<int>((static_cast<long long>(p.units) * n_pad + gridDim.x - 1) / gridDim.x)
                      : p.tiles_per_split;
    } else {
        chunk = max(split_tiles(p, total_tiles), 1);
        n_pad = chunk * p.splits;
    }
    const long long work_total = static_cast<long long>(p.units) * n_pad;
    long long work = static_cast<long long>(blockIdx.x) * chunk;
    const long long work_end = min(work_total, work + chunk);
    // a device-side token count beyond the buffers is cut to the token stride: tell the host
    if (p.dyn && blockIdx.x == 0 && tid == 0 && p.dyn[2] > p.tok_stride) atomicOr(p.status, RESKV_STATUS_STATE_RANGE);
    if (work >= work_end) return;

    if (tid == 0) {
        timed_out = 0;
        for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[s], ML::kPad ? 1 + kThreadsM : 1);
        mbar_fence_init();
    }

    // ---- once per CTA: sin/cos of (tile offset j) x (frequency i) ------------------------------
    {
        const int i = tid & 63, half = tid >> 6;
        const float f = rope_freq(p.inv_freq, p.theta, i);
        {
            const int j0 = half * 32;
            float s, c, s1, c1;
            sincosf(static_cast<float>(j0) * f, &s, &c);
            sincosf(f, &s1, &c1);
            for (int j = j0; j < j0 + 32; ++j) {
                trig[trig_index(j, i)] = make_float2(c, s);
                const float ns = s * c1 + c * s1, nc = c * c1 - s * s1;
                s = ns, c = nc;
            }
        }
    }
    // query items of this thread: (head, two adjacent frequencies i2, i2 + 1); the per-tile angle step
    // does not depend on the unit
    float q_f[kItems][2], dn_c[kItems][2], dn_s[kItems][2];
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
        const int i2 = ((tid + it * kThreadsM) & 31) * 2;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            q_f[it][u] = rope_freq(p.inv_freq, p.theta, i2 + u);
            sincosf(static_cast<float>(kTileM) * q_f[it][u], &dn_s[it][u], &dn_c[it][u]);
        }
    }
    __syncthreads();  // barriers initialised, sin/cos table complete

    // sin/cos of this lane's two rows (tile offsets 16 warp + g and + 8) and 16 frequencies: the
    // same in every tile, so they live in registers for the whole kernel
    float4 trA_r[8], trB_r[8];
    {
        const int tokA = warp * 16 + g, tokB = tokA + 8;
        const float4* trA = reinterpret_cast<const float4*>(trig + tokA * kTrigStride);
        const float4* trB = reinterpret_cast<const float4*>(trig + tokB * kTrigStride);
        const int tr_swz = (tokA & 1) << 2;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            trA_r[u] = trA[(u * 4 + qd) ^ tr_swz];
            trB_r[u] = trB[(u * 4 + qd) ^ tr_swz];
        }
    }

    __syncthreads();  // every lane has its sin/cos values: the table's memory becomes the ring of stages
    const float q_mul = p.scaling * kLog2e;
    uint2* pre_k = pre + warp * 32;
    uint2* pre_v = pre_k + 16;
    uint32_t ring = 0;  // tiles issued / consumed so far by this CTA (ring slot and barrier phase follow it)
    bool lost = false;
    bool first_segment = true;

    while (work < work_end) {
        // ---- the segment: unit, its tile range, its partial slot --------------------------------
        const int unit = static_cast<int>(work / n_pad);
        const int t_pad = static_cast<int>(work - static_cast<long long>(unit) * n_pad);
        const int len = static_cast<int>(min(static_cast<long long>(n_pad - t_pad), work_end - work));
        const int tile_begin = min(t_pad, total_tiles);
        const int ntiles = max(0, min(total_tiles, t_pad + len) - tile_begin);
        const int slot = static_cast<int>(blockIdx.x) - static_cast<int>((static_cast<long long>(unit) * n_pad) / chunk);
        const bool closes_unit = t_pad + len == n_pad;
        work += len;
        const int b = unit / p.kh, hkv = unit % p.kh;

        const size_t unit_tok = static_cast<size_t>(unit) * p.tok_stride;
        const unsigned char* km_g = static_cast<const unsigned char*>(p.kb) + unit_tok * ML::kMetaBytes;
        const unsigned char* vm_g = static_cast<const unsigned char*>(p.vb) + unit_tok * ML::kMetaBytes;
        const unsigned char* kp_g = static_cast<const unsigned char*>(p.kp) + unit_tok * ML::kPayloadBytes;
        const unsigned char* vp_g = static_cast<const unsigned char*>(p.vp) + unit_tok * ML::kPayloadBytes;
        const int8_t* kid_g = p.kid + unit_tok;
        const int8_t* vid_g = p.vid + unit_tok;
        const __half* ks_g = ML::kScale ? p.ks + unit_tok : nullptr;
        const __half* vs_g = ML::kScale ? p.vs + unit_tok : nullptr;

        // the previous segment's epilogue still reads the stage memory and the centroid table
        if (!first_segment) __syncthreads();
        first_segment = false;

        auto issue = [&](int tile_rel) {
            const int t0 = (tile_begin + tile_rel) * kTileM;
            const int n = min(kTileM, tokens - t0);
            const uint32_t ring_slot = (ring + tile_rel) % kStages;
            StageT& st = stages[ring_slot];
            uint64_t* bar = &full_bar[ring_slot];
            // 8-byte metadata rows stay bulk-copyable: tiles start at multiples of 64 tokens and the host
            // selects this kernel for them only when token count and token stride are even
            const uint32_t md_bytes = n * ML::kMetaBytes, pl_bytes = n * ML::kPayloadBytes;
            const unsigned char* kp_src = kp_g + static_cast<size_t>(t0) * ML::kPayloadBytes;
            const unsigned char* vp_src = vp_g + static_cast<size_t>(t0) * ML::kPayloadBytes;
            if constexpr (ML::kPad != 0) {
                // metadata in bulk by one thread; payload rows in 16-byte pieces by everyone, into padded rows
                if (tid == 0) {
                    mbar_arrive_expect_tx(bar, 2 * md_bytes);
                    bulk_g2s(st.km, km_g + static_cast<size_t>(t0) * ML::kMetaBytes, md_bytes, bar);
                    bulk_g2s(st.vm, vm_g + static_cast<size_t>(t0) * ML::kMetaBytes, md_bytes, bar);
                }
                constexpr int kPieces = ML::kPayloadBytes / 16, kRow = ML::kPayloadBytes + ML::kPad;
                for (int c = tid; c < n * kPieces; c += kThreadsM) {
                    const int dst = (c / kPieces) * kRow + (c % kPieces) * 16;
                    cp_async16(st.kp + dst, kp_src + c * 16);
                    cp_async16(st.vp + dst, vp_src + c * 16);
                }
                cp_async_arrive(bar);
            } else if (tid == 0) {
                mbar_arrive_expect_tx(bar, 2 * md_bytes + 2 * pl_bytes);
                if (ML::kMetaBytes) {
                    bulk_g2s(st.km, km_g + static_cast<size_t>(t0) * ML::kMetaBytes, md_bytes, bar);
                    bulk_g2s(st.vm, vm_g + static_cast<size_t>(t0) * ML::kMetaBytes, md_bytes, bar);
                }
                bulk_g2s(st.kp, kp_src, pl_bytes, bar);
                bulk_g2s(st.vp, vp_src, pl_bytes, bar);
            }
        };
        for (int s = 0; s < kStages && s < ntiles; ++s) issue(s);

        // ---- per unit: key centroids (FP32, swizzled rows) ---------------------------------------
        {
            const __half* src = p.kc + static_cast<size_t>(unit) * p.ck * kHeadDim;
            for (int idx = tid; idx < p.ck * (kHeadDim / 8); idx += kThreadsM) {  // 8 coordinates per step
                const int row = idx / (kHeadDim / 8), d = (idx % (kHeadDim / 8)) * 8;
                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src + row * kHeadDim + d));
                const __half2* h = reinterpret_cast<const __half2*>(&raw);
                const float2 v0 = __half22float2(h[0]), v1 = __half22float2(h[1]), v2 = __half22float2(h[2]), v3 = __half22float2(h[3]);
                *reinterpret_cast<float4*>(kc_s + row * kCenStride + cen_index(d)) = make_float4(v0.x, v0.y, v1.x, v1.y);
                *reinterpret_cast<float4*>(kc_s + row * kCenStride + cen_index(d + 4)) = make_float4(v2.x, v2.y, v3.x, v3.y);
            }
        }

        // ---- query state: angle (pos_q - P0) * f goes down by 64 f per tile; seeded exactly every
        // kReseedTiles tiles ------------------------------------------------------------------------
        float q_lo[kItems][2], q_hi[kItems][2], st_c[kItems][2], st_s[kItems][2];
#pragma unroll
        for (int it = 0; it < kItems; ++it) {
            const int item = tid + it * kThreadsM;
            const int h = item >> 5, i2 = (item & 31) * 2;
            const bool on = item < GQA * 32;
            const __half* qrow = p.q + (static_cast<size_t>(b) * p.nh + hkv * GQA + (on ? h : 0)) * kHeadDim;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                q_lo[it][u] = on ? __half2float(qrow[i2 + u]) * q_mul : 0.f;
                q_hi[it][u] = on ? __half2float(qrow[i2 + u + 64]) * q_mul : 0.f;
                st_c[it][u] = 1.f, st_s[it][u] = 0.f;
            }
        }

        auto write_query = [&](int tile_rel) {
            // Qt = R(pos_q - P0) q  for the tile that starts at token t0, as FP16 hi + lo
            const int t0 = (tile_begin + tile_rel) * kTileM;
            __half* base = qf + (tile_rel & 1) * (kQSets * GQA * kQStride);
#pragma unroll
            for (int it = 0; it < kItems; ++it) {
                const int item = tid + it * kThreadsM;
                if (item >= GQA * 32) continue;
                const int h = item >> 5, i2 = (item & 31) * 2;
                float lo[2], hi[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (tile_rel % kReseedTiles == 0) {
                        const float delta = static_cast<float>(query_position(p) - (p.start_pos + t0));
                        sincosf(delta * q_f[it][u], &st_s[it][u], &st_c[it][u]);
                    }
                    const float c = st_c[it][u], s = st_s[it][u];
                    lo[u] = q_lo[it][u] * c - q_hi[it][u] * s;
                    hi[u] = q_hi[it][u] * c + q_lo[it][u] * s;
                    // next tile: angle - 64 f
                    st_c[it][u] = c * dn_c[it][u] + s * dn_s[it][u];
                    st_s[it][u] = s * dn_c[it][u] - c * dn_s[it][u];
                }
                const __half2 lo_h = __floats2half2_rn(lo[0], lo[1]), hi_h = __floats2half2_rn(hi[0], hi[1]);
                const float2 lo_f = __half22float2(lo_h), hi_f = __half22float2(hi_h);
                __half* row_hi = base + h * kQStride;
                __half* row_lo = base + (GQA + h) * kQStride;
                *reinterpret_cast<__half2*>(row_hi + i2) = lo_h;
                *reinterpret_cast<__half2*>(row_hi + i2 + 64) = hi_h;
                *reinterpret_cast<__half2*>(row_lo + i2) = __floats2half2_rn(lo[0] - lo_f.x, lo[1] - lo_f.y);
                *reinterpret_cast<__half2*>(row_lo + i2 + 64) = __floats2half2_rn(hi[0] - hi_f.x, hi[1] - hi_f.y);
            }
        };
        if (ntiles > 0) write_query(0);

        // ---- per-warp running state -------------------------------------------------------------
        float acc[8][4];          // O^T: m-block i -> coordinates 16g+2i (c0,c1) and 16g+2i+1 (c2,c3); heads 2q, 2q+1
        float m_used[2], l_part[2];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        m_used[0] = m_used[1] = -INFINITY;
        l_part[0] = l_part[1] = 0.f;
        // cluster mass beta[value cluster][head] of this warp's tokens, accumulated by the tensor cores as
        // onehot(value id)^T . P: rows = clusters 16 mb + g (+ 8), columns = heads 2q, 2q + 1
        float bacc[BETA][4];
#pragma unroll
        for (int mb = 0; mb < BETA; ++mb) bacc[mb][0] = bacc[mb][1] = bacc[mb][2] = bacc[mb][3] = 0.f;

        // cluster ids (and FP16 scales) of this warp's 16 tokens of the next tile: lanes 0..15 hold the
        // key side of token `lane`, lanes 16..31 the value side of token `lane - 16`
        auto load_ids = [&](int tile_rel, int& id, uint32_t& scale) {
            const int t = (tile_begin + tile_rel) * kTileM + warp * 16 + (lane & 15);
            id = 0, scale = 0u;
            if (tile_rel < ntiles && t < tokens) {
                // volatile: issue the loads here, a whole tile ahead of their use, instead of letting the
                // compiler sink them next to the consumer
                const int8_t* src = ((lane < 16) ? kid_g : vid_g) + t;
                asm volatile("ld.global.nc.s8 %0, [%1];" : "=r"(id) : "l"(src));
                if constexpr (ML::kScale) {
                    const __half* ssrc = ((lane < 16) ? ks_g : vs_g) + t;
                    unsigned short h;
                    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(h) : "l"(ssrc));
                    scale = h;
                }
            }
        };
        int ids_next;
        uint32_t scl_next;
        load_ids(0, ids_next, scl_next);
        __syncthreads();  // centroid table and first query tile ready

        for (int it = 0; it < ntiles; ++it) {
            const int t0 = (tile_begin + it) * kTileM;
            const int ids_cur = ids_next;
            const uint32_t scl_cur = scl_next;
            load_ids(it + 1, ids_next, scl_next);
            const uint32_t ring_it = ring + it;
            if (!mbar_wait(&full_bar[ring_it % kStages], (ring_it / kStages) & 1)) lost = true;
            const StageT& st = stages[ring_it % kStages];
            const int nvalid = min(16, tokens - (t0 + warp * 16));  // valid tokens of this warp's block
            if (nvalid > 0) {
                if constexpr (ML::kPrefix) {
                    // rank bases of the block's 16 key bitmaps (lanes 0..15) and value bitmaps (16..31)
                    const int tok = warp * 16 + (lane & 15);
                    const uint4 bm = reinterpret_cast<const uint4*>((lane < 16) ? st.km : st.vm)[tok];
                    pre_k[lane] = rank_bases(bm);  // pre_v == pre_k + 16
                    __syncwarp();
                }

                // ================= keys: rows g and g + 8 of the block =================
                const int tokA = warp * 16 + g, tokB = tokA + 8;
                const bool okA = g < nvalid, okB = g + 8 < nvalid;
                const int kidA = min(max(__shfl_sync(0xffffffffu, ids_cur, g), 0), p.ck - 1);
                const int kidB = min(max(__shfl_sync(0xffffffffu, ids_cur, g + 8), 0), p.ck - 1);
                const unsigned char* pk_bytes = reinterpret_cast<const unsigned char*>(pre_k);
                Field fAl = ML::field(st.kp, st.km, pk_bytes, tokA, qd, okA), fAh = ML::field(st.kp, st.km, pk_bytes, tokA, 4 + qd, okA);
                Field fBl = ML::field(st.kp, st.km, pk_bytes, tokB, qd, okB), fBh = ML::field(st.kp, st.km, pk_bytes, tokB, 4 + qd, okB);
                const unsigned short kscA = static_cast<unsigned short>(__shfl_sync(0xffffffffu, scl_cur, g));
                const unsigned short kscB = static_cast<unsigned short>(__shfl_sync(0xffffffffu, scl_cur, g + 8));
                // FP32 centroid rows; the lane's low field starts at 16q, its partner field at 64 + 16q
                const float* cA = kc_s + kidA * kCenStride + 16 * qd;
                const float* cB = kc_s + kidB * kCenStride + 16 * qd;
                const int cen_swz = (qd >> 1) & 1;  // 16-byte unit swap of this lane's fields
                const __half* qbuf = qf + (it & 1) * (kQSets * GQA * kQStride) + g * kQStride + 16 * qd;
                // rows of the B operand: the real heads (hi halves), then -- packed form -- their lo halves
                const bool q_on = g < (kPackQ ? 2 * GQA : GQA);

                // independent accumulators (hi.hi, hi.lo, lo.hi) keep the MMA dependency chains short
                float sc[4] = {0.f, 0.f, 0.f, 0.f}, sc2[4] = {0.f, 0.f, 0.f, 0.f}, sc3[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    // four coordinates 16q + 4ks .. +3 and their partners + 64, both tokens:
                    // k = centroid (+ residual where the bitmap bit is set)
                    // query fragments of k-step ks (low half of the head) and ks + 4 (high half), requested first
                    uint2 qh_l = make_uint2(0u, 0u), qh_h = qh_l, ql_l = qh_l, ql_h = qh_l;
                    if (q_on) {
                        qh_l = *reinterpret_cast<const uint2*>(qbuf + 4 * ks);
                        qh_h = *reinterpret_cast<const uint2*>(qbuf + 64 + 4 * ks);
                        if constexpr (!kPackQ) {
                            ql_l = *reinterpret_cast<const uint2*>(qbuf + GQA * kQStride + 4 * ks);
                            ql_h = *reinterpret_cast<const uint2*>(qbuf + GQA * kQStride + 64 + 4 * ks);
                        }
                    }
                    const int cu = (ks ^ cen_swz) * 4;
                    const float4 al = *reinterpret_cast<const float4*>(cA + cu), ah = *reinterpret_cast<const float4*>(cA + 64 + cu);
                    const float4 bl = *reinterpret_cast<const float4*>(cB + cu), bh = *reinterpret_cast<const float4*>(cB + 64 + cu);
                    float kAl[4] = {al.x, al.y, al.z, al.w}, kAh[4] = {ah.x, ah.y, ah.z, ah.w};
                    float kBl[4] = {bl.x, bl.y, bl.z, bl.w}, kBh[4] = {bh.x, bh.y, bh.z, bh.w};
                    if constexpr (Field::kSlotwise) {
                        // the four walks advance together, one coordinate each at a time
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            fAl.add1(4 * ks + e, kAl[e]);
                            fAh.add1(4 * ks + e, kAh[e]);
                            fBl.add1(4 * ks + e, kBl[e]);
                            fBh.add1(4 * ks + e, kBh[e]);
                        }
                    } else {
                        fAl.add4(ks, kAl, kscA);
                        fAh.add4(ks, kAh, kscA);
                        fBl.add4(ks, kBl, kscB);
                        fBh.add4(ks, kBh, kscB);
                    }
                    float rAl[4], rAh[4], rBl[4], rBh[4];
#pragma unroll
                    for (int e2 = 0; e2 < 2; ++e2) {
                        const float4 ta = trA_r[ks * 2 + e2];  // (cos, sin) of two neighbouring frequencies
                        const float4 tb = trB_r[ks * 2 + e2];
                        const int e = 2 * e2;
                        rAl[e] = kAl[e] * ta.x - kAh[e] * ta.y;
                        rAh[e] = kAh[e] * ta.x + kAl[e] * ta.y;
                        rAl[e + 1] = kAl[e + 1] * ta.z - kAh[e + 1] * ta.w;
                        rAh[e + 1] = kAh[e + 1] * ta.z + kAl[e + 1] * ta.w;
                        rBl[e] = kBl[e] * tb.x - kBh[e] * tb.y;
                        rBh[e] = kBh[e] * tb.x + kBl[e] * tb.y;
                        rBl[e + 1] = kBl[e + 1] * tb.z - kBh[e + 1] * tb.w;
                        rBh[e + 1] = kBh[e + 1] * tb.z + kBl[e + 1] * tb.w;
                    }
                    uint32_t a0, a1, a2, a3, l0, l1, l2, l3;
                    split_h2(rAl[0], rAl[1], a0, l0);
                    split_h2(rBl[0], rBl[1], a1, l1);
                    split_h2(rAl[2], rAl[3], a2, l2);
                    split_h2(rBl[2], rBl[3], a3, l3);
                    mma_16816(sc, a0, a1, a2, a3, qh_l.x, qh_l.y);
                    if constexpr (!kPackQ) mma_16816(sc2, a0, a1, a2, a3, ql_l.x, ql_l.y);
                    mma_16816(sc3, l0, l1, l2, l3, qh_l.x, qh_l.y);
                    split_h2(rAh[0], rAh[1], a0, l0);
                    split_h2(rBh[0], rBh[1], a1, l1);
                    split_h2(rAh[2], rAh[3], a2, l2);
                    split_h2(rBh[2], rBh[3], a3, l3);
                    mma_16816(sc, a0, a1, a2, a3, qh_h.x, qh_h.y);
                    if constexpr (!kPackQ) mma_16816(sc2, a0, a1, a2, a3, ql_h.x, ql_h.y);
                    mma_16816(sc3, l0, l1, l2, l3, qh_h.x, qh_h.y);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) sc[i] += sc2[i] + sc3[i];
                if constexpr (kPackQ) {
                    // columns h (query hi) and h + 4 (query lo) of a head sit in lanes q and q ^ 2; afterwards
                    // lanes q = 2, 3 repeat heads 0..3 (their results are never stored)
#pragma unroll
                    for (int i = 0; i < 4; ++i) sc[i] += __shfl_xor_sync(0xffffffffu, sc[i], 2);
                }
                // value fields of tokens 2q, 2q+1, 2q+8, 2q+9, coordinates [16g, 16g+16): set up before the softmax so
                // that their mask and rank-base loads are in flight during it
                const unsigned char* pv_bytes = reinterpret_cast<const unsigned char*>(pre_v);
                const int r0 = 2 * qd, r1 = 2 * qd + 1, r2 = 2 * qd + 8, r3 = 2 * qd + 9;
                Field f0 = ML::field(st.vp, st.vm, pv_bytes, warp * 16 + r0, g, r0 < nvalid);
                Field f1 = ML::field(st.vp, st.vm, pv_bytes, warp * 16 + r1, g, r1 < nvalid);
                Field f2 = ML::field(st.vp, st.vm, pv_bytes, warp * 16 + r2, g, r2 < nvalid);
                Field f3 = ML::field(st.vp, st.vm, pv_bytes, warp * 16 + r3, g, r3 < nvalid);

                // sc: c0,c1 = (token g, heads 2q, 2q+1), c2,c3 = (token g+8, ...), log2 domain
                if (!okA) sc[0] = sc[1] = -INFINITY;
                if (!okB) sc[2] = sc[3] = -INFINITY;

                // ================= softmax (lazy running maximum) =================
                float mt[2] = {fmaxf(sc[0], sc[2]), fmaxf(sc[1], sc[3])};
#pragma unroll
                for (int off = 4; off < 32; off <<= 1) {
                    mt[0] = fmaxf(mt[0], __shfl_xor_sync(0xffffffffu, mt[0], off));
                    mt[1] = fmaxf(mt[1], __shfl_xor_sync(0xffffffffu, mt[1], off));
                }
                const bool grow = mt[0] > m_used[0] + kRescaleThreshold || mt[1] > m_used[1] + kRescaleThreshold;
                if (__any_sync(0xffffffffu, grow)) {
                    float alpha[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const float m_new = fmaxf(m_used[u], mt[u]);
                        alpha[u] = (m_used[u] == -INFINITY) ? 0.f : fast_exp2(m_used[u] - m_new);
                        m_used[u] = m_new;
                        l_part[u] *= alpha[u];
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        acc[i][0] *= alpha[0], acc[i][2] *= alpha[0];
                        acc[i][1] *= alpha[1], acc[i][3] *= alpha[1];
                    }
#pragma unroll
                    for (int mb = 0; mb < BETA; ++mb) {
                        bacc[mb][0] *= alpha[0], bacc[mb][2] *= alpha[0];
                        bacc[mb][1] *= alpha[1], bacc[mb][3] *= alpha[1];
                    }
                }
                float pr[4];
                pr[0] = fast_exp2(sc[0] - m_used[0]), pr[1] = fast_exp2(sc[1] - m_used[1]);
                pr[2] = fast_exp2(sc[2] - m_used[0]), pr[3] = fast_exp2(sc[3] - m_used[1]);
                __half2 p01 = __floats2half2_rn(pr[0], pr[1]), p23 = __floats2half2_rn(pr[2], pr[3]);
                const float2 p01f = __half22float2(p01), p23f = __half22float2(p23);
                l_part[0] += p01f.x + p23f.x;
                l_part[1] += p01f.y + p23f.y;
                // P as B operand (tokens x heads): transpose the two 8x8 halves
                uint32_t pb0 = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&p01));
                uint32_t pb1 = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&p23));
                {
                    // cluster mass: one-hot rows A[c][t] = (value id of token t == c), built two tokens at a
                    // time by a packed FP16 compare; tokens beyond the end have p = 0
                    const int w0 = __shfl_sync(0xffffffffu, ids_cur, 16 + 2 * qd), w1 = __shfl_sync(0xffffffffu, ids_cur, 17 + 2 * qd);
                    const int w2 = __shfl_sync(0xffffffffu, ids_cur, 24 + 2 * qd), w3 = __shfl_sync(0xffffffffu, ids_cur, 25 + 2 * qd);
                    const __half2 gg = __half2half2(__int2half_rn(g));
                    const __half2 d01 = __hsub2(__halves2half2(__int2half_rn(w0), __int2half_rn(w1)), gg);
                    const __half2 d23 = __hsub2(__halves2half2(__int2half_rn(w2), __int2half_rn(w3)), gg);
#pragma unroll
                    for (int mb = 0; mb < BETA; ++mb) {
                        if (16 * mb < p.cv) {
                            const __half2 lo = __float2half2_rn(16.f * mb), hi = __float2half2_rn(16.f * mb + 8.f);
                            const __half2 a0 = __heq2(d01, lo), a1 = __heq2(d01, hi), a2 = __heq2(d23, lo), a3 = __heq2(d23, hi);
#ifdef RESKV_ABLATE_ACCUMULATORS
                            mma_16816(bacc[0], *reinterpret_cast<const uint32_t*>(&a0), *reinterpret_cast<const uint32_t*>(&a1),
#else
                            mma_16816(bacc[mb], *reinterpret_cast<const uint32_t*>(&a0), *reinterpret_cast<const uint32_t*>(&a1),
#endif
                                      *reinterpret_cast<const uint32_t*>(&a2), *reinterpret_cast<const uint32_t*>(&a3), pb0, pb1);
                        }
                    }
                }
                if constexpr (ML::kScaleP) {
                    // quantised values enter the MMA as integer codes: their per-token scale rides on P
                    const float vsA = h2f_bits(__shfl_sync(0xffffffffu, scl_cur, 16 + g));
                    const float vsB = h2f_bits(__shfl_sync(0xffffffffu, scl_cur, 24 + g));
                    p01 = __floats2half2_rn(p01f.x * vsA, p01f.y * vsA);
                    p23 = __floats2half2_rn(p23f.x * vsB, p23f.y * vsB);
                    pb0 = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&p01));
                    pb1 = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&p23));
                }

                // O^T += Vres^T . P.  Values: tokens 2q, 2q+1, 2q+8, 2q+9 of the block, coordinates [16g, 16g+16);
                // m-block i holds coordinates 16g + 2i (rows g) and 16g + 2i + 1 (rows g + 8), so that the MMAs
                // follow the field walks two coordinates at a time
                {
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        uint32_t h0[4], h1[4], h2[4], h3[4];
                        if constexpr (Field::kSlotwise) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                h0[e] = f0.bits1(4 * ks + e);
                                h1[e] = f1.bits1(4 * ks + e);
                                h2[e] = f2.bits1(4 * ks + e);
                                h3[e] = f3.bits1(4 * ks + e);
                            }
                        } else {
                            f0.bits4(ks, h0);
                            f1.bits4(ks, h1);
                            f2.bits4(ks, h2);
                            f3.bits4(ks, h3);
                        }
#ifdef RESKV_ABLATE_ACCUMULATORS  // timing experiment only (wrong results): all value MMAs add into one accumulator
                        mma_16816(acc[0], h0[0] | (h1[0] << 16), h0[1] | (h1[1] << 16), h2[0] | (h3[0] << 16),
                                  h2[1] | (h3[1] << 16), pb0, pb1);
                        mma_16816(acc[0], h0[2] | (h1[2] << 16), h0[3] | (h1[3] << 16), h2[2] | (h3[2] << 16),
                                  h2[3] | (h3[3] << 16), pb0, pb1);
#else
                        mma_16816(acc[2 * ks], h0[0] | (h1[0] << 16), h0[1] | (h1[1] << 16), h2[0] | (h3[0] << 16),
                                  h2[1] | (h3[1] << 16), pb0, pb1);
                        mma_16816(acc[2 * ks + 1], h0[2] | (h1[2] << 16), h0[3] | (h1[3] << 16), h2[2] | (h3[2] << 16),
                                  h2[3] | (h3[3] << 16), pb0, pb1);
#endif
                    }
                }
                __syncwarp();  // rank-base table is rewritten next tile
            }
            if (it + 1 < ntiles) write_query(it + 1);
            __syncthreads();  // ring slot free, next query tile visible
            if (it + kStages < ntiles) issue(it + kStages);
        }
        ring += static_cast<uint32_t>(ntiles);

        // ---- combine warps, write the segment's partial -------------------------------------------
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l_part[0] += __shfl_xor_sync(0xffffffffu, l_part[0], off);
            l_part[1] += __shfl_xor_sync(0xffffffffu, l_part[1], off);
        }
        if (g == 0) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int h = 2 * qd + u;
                if (h < GQA) red_m[h][warp] = m_used[u], red_l[h][warp] = l_part[u];
            }
        }
        __syncthreads();
        float* red_acc = reinterpret_cast<float*>(smem_raw);  // [warps][GQA][128], stage memory is free now
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int h = 2 * qd + u;
            if (h < GQA) {
                float fm = red_m[h][0];
#pragma unroll
                for (int w = 1; w < kWarpsM; ++w) fm = fmaxf(fm, red_m[h][w]);
                const float scale = (m_used[u] == -INFINITY) ? 0.f : fast_exp2(m_used[u] - fm);
                float* dst = red_acc + (warp * GQA + h) * kHeadDim + 16 * g;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    dst[2 * i] = acc[i][u] * scale;
                    dst[2 * i + 1] = acc[i][2 + u] * scale;
                }
                float* bdst = beta_s + (warp * GQA + h) * kMaxClusters + g;
#pragma unroll
                for (int mb = 0; mb < 4; ++mb) {
                    bdst[16 * mb] = mb < BETA ? bacc[mb < BETA ? mb : 0][u] : 0.f;
                    bdst[16 * mb + 8] = mb < BETA ? bacc[mb < BETA ? mb : 0][2 + u] : 0.f;
                }
            }
        }
        __syncthreads();
        const size_t part = static_cast<size_t>(b) * p.nh + hkv * GQA;
        if (slot >= 0 && slot < p.splits) {
            for (int idx = tid; idx < GQA * kHeadDim; idx += kThreadsM) {
                const int h = idx / kHeadDim, d = idx % kHeadDim;
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < kWarpsM; ++w) sum += red_acc[(w * GQA + h) * kHeadDim + d];
                p.ws_delta[((part + h) * p.splits + slot) * kHeadDim + d] = sum;
            }
            for (int idx = tid; idx < GQA * kMaxClusters; idx += kThreadsM) {
                const int h = idx / kMaxClusters, c = idx % kMaxClusters;
                float fm = red_m[h][0];
#pragma unroll
                for (int w = 1; w < kWarpsM; ++w) fm = fmaxf(fm, red_m[h][w]);
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < kWarpsM; ++w) {
                    const float scale = (red_m[h][w] == -INFINITY) ? 0.f : fast_exp2(red_m[h][w] - fm);
                    sum += beta_s[(w * GQA + h) * kMaxClusters + c] * scale;
                }
                p.ws_beta[((part + h) * p.splits + slot) * kMaxClusters + c] = sum;
            }
            if (tid < GQA) {
                const int h = tid;
                float fm = red_m[h][0];
                for (int w = 1; w < kWarpsM; ++w) fm = fmaxf(fm, red_m[h][w]);
                float fl = 0.f;
                for (int w = 0; w < kWarpsM; ++w)
                    fl += (red_m[h][w] == -INFINITY) ? 0.f : red_l[h][w] * fast_exp2(red_m[h][w] - fm);
                p.ws_m[(part + h) * p.splits + slot] = fm;
                p.ws_l[(part + h) * p.splits + slot] = fl;
            }
            // the segment that ends its unit marks the unit's unused slots as empty
            if (closes_unit) {
                for (int idx = tid; idx < GQA * (p.splits - slot - 1); idx += kThreadsM) {
                    const int h = idx % GQA, s = slot + 1 + idx / GQA;
                    p.ws_m[(part + h) * p.splits + s] = -INFINITY;
                    p.ws_l[(part + h) * p.splits + s] = 0.f;
                }
            }
        } else if (tid == 0) {
            atomicOr(p.status, RESKV_STATUS_STATE_RANGE);
        }
    }
    if (lost && lane == 0) atomicOr(&timed_out, 1u);
    __syncthreads();
    if (tid == 0 && timed_out) atomicOr(p.status, RESKV_STATUS_WAIT_TIMEOUT);
}

}  // namespace mma

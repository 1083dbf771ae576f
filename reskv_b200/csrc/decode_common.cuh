// Definitions shared by the decode translation units.
#pragma once

#include "common.cuh"

namespace reskv {

struct DecodeParams;
// Launches the tensor-core partial kernel of a non-bitmap layout (decode_packed_mma.cu).
// layout: 0 = INT4, 1 = INT2 (unstructured), 2 = tiled FP16, 3 = structured FP16, 4 = structured INT4,
// 5 / 6 = compact INT4 with 64 / 32 codes, 7 = compact INT2 with 64 codes.
int launch_packed_mma(const DecodeParams& p, int layout, int gqa, int units, cudaStream_t stream);

namespace {

constexpr int kTile = 64;    // tokens per pipeline stage
constexpr int kWarps = 8;    // warps per CTA
constexpr int kThreads = kWarps * 32;
constexpr int kTokPerWarp = kTile / kWarps;
constexpr int kReseedTiles = 16;
constexpr int kWsHeader = 256;  // bytes reserved at the start of the workspace (status word)

}  // namespace

struct DecodeParams {
    const __half* q;
    const __half* kc;
    const int8_t* kid;
    const void* kp;   // payload rows
    const void* kb;   // metadata rows (bitmaps, tile masks / indices) or null
    const int8_t* vid;
    const void* vp;
    const void* vb;
    const __half* ks;  // per-token scales of quantised layouts or null
    const __half* vs;
    float* ws_m;
    float* ws_l;
    float* ws_delta;
    float* ws_beta;
    uint32_t* status;
    const float* inv_freq;
    int64_t tok_stride;
    int kh, nh, tokens, ck, cv;
    // splits = partial slots per query head in the workspace; tiles_per_split = tiles per CTA (see `balanced`)
    int start_pos, pos_q, splits, tiles_per_split;
    // units = batch * kv heads.  balanced != 0: the tensor-core kernel runs a 1-D grid whose CTAs each take an
    // equal share of all units' tiles (a CTA may finish one unit and start the next); balanced == 0: one CTA per
    // (unit, split) with `tiles_per_split` tiles each.
    int units, balanced, grid;  // grid = CTAs of the tensor-core kernel
    float theta, scaling;
    // optional device-resident step state {query position, dense-window tokens, compressed tokens
    // or -1, reserved}: when set it overrides pos_q, the merge kernel's recent-token count and
    // (third word, if not negative) `tokens`, so that a captured CUDA graph can be replayed for
    // consecutive decode steps and across group compressions
    const int32_t* dyn;
};

// compressed tokens of this launch: from the device step state when it carries a count
__device__ __forceinline__ int token_count(const DecodeParams& p) {
    if (p.dyn) {
        const int t = p.dyn[2];
        if (t >= 0) return static_cast<int>(min(static_cast<int64_t>(t), p.tok_stride));
    }
    return p.tokens;
}

// tiles per split: the host's figure, or the same formula on the device-side token count
__device__ __forceinline__ int split_tiles(const DecodeParams& p, int total_tiles) {
    return p.dyn ? (total_tiles + p.splits - 1) / p.splits : p.tiles_per_split;
}

// query position of this launch: from the device step state when one is attached
__device__ __forceinline__ int query_position(const DecodeParams& p) { return p.dyn ? p.dyn[0] : p.pos_q; }

namespace {

__device__ __forceinline__ float rope_freq(const float* inv_freq, float theta, int i) {
    return inv_freq ? inv_freq[i] : powf(theta, -static_cast<float>(i) / 64.0f);
}

}  // namespace
}  // namespace reskv

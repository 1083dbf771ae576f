// One decode group (the oldest `group` tokens of the dense window) appended to a compressed cache in place, and the
// window slide that follows it.
//
// The host-side sequence this replaces is, per layer and for K and V each: incremental clustering (new centroid
// table + ids), packing into fresh tensors, six slice copies into the capacity buffers, three slice copies that move
// the window's remaining tokens to the front.  The device work of all that is ~0.1 ms; issued as ~15 separate tensor
// operations it costs ~0.45 ms of host time per layer at every batch size.  Here it is two calls.
#include "common.cuh"

namespace reskv {
namespace {

constexpr int kNarrowThreads = 256;

// ids int32 [units, tokens] of K and of V -> int8 rows `stride` tokens apart, behind the live tokens
__global__ void narrow_ids_kernel(const int32_t* k_ids, const int32_t* v_ids, int8_t* k_dst, int8_t* v_dst,
                                  int tokens, int64_t k_stride, int64_t v_stride, int total) {
    const int i = blockIdx.x * kNarrowThreads + threadIdx.x;
    if (i >= total) return;
    const int unit = i / tokens, t = i % tokens;
    k_dst[static_cast<size_t>(unit) * k_stride + t] = static_cast<int8_t>(k_ids[i]);
    v_dst[static_cast<size_t>(unit) * v_stride + t] = static_cast<int8_t>(v_ids[i]);
}

// grid = (units, 3 buffers), 128 threads = 8 tokens x 16 pieces of 16 bytes per pass.  Tokens [src, src + count) of a
// unit move to [dst, dst + count), dst < src.  Every pass reads its tokens before any thread writes (a barrier in
// between) and passes go upwards, so overlapping ranges are moved correctly.
__global__ void __launch_bounds__(128) window_shift_kernel(uint4* win_k, uint4* win_raw, uint4* win_v, int capacity,
                                                           int dst, int src, int count) {
    uint4* buf = blockIdx.y == 0 ? win_k : blockIdx.y == 1 ? win_raw : win_v;
    buf += static_cast<size_t>(blockIdx.x) * capacity * (kHeadDim / 8);
    const int row = threadIdx.x >> 4, piece = threadIdx.x & 15;
    for (int t0 = 0; t0 < count; t0 += 8) {
        const int t = t0 + row;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (t < count) v = buf[static_cast<size_t>(src + t) * (kHeadDim / 8) + piece];
        __syncthreads();
        if (t < count) buf[static_cast<size_t>(dst + t) * (kHeadDim / 8) + piece] = v;
        __syncthreads();
    }
}

struct Side {
    const void* x;
    const void* old_centroids;
    int old_clusters;
    void* new_centroids;
    int new_clusters;
    void* ids;      // int8 [units, stride]
    void* payload;  // rows of the arena, all starting at token 0
    void* meta;
    void* scale;
    int64_t stride;
};

size_t payload_row_bytes(int layout, int bits, int nnz) {
    if (bits == 16) return static_cast<size_t>(nnz) * 2;
    if (layout == RESKV_LAYOUT_COMPACT) return static_cast<size_t>(nnz) * bits / 8;
    return layout == RESKV_LAYOUT_STRUCTURED ? 16 : static_cast<size_t>(16) * bits;
}

size_t meta_row_bytes(int layout, int bits) {
    if (layout == RESKV_LAYOUT_UNSTRUCTURED) return bits == 16 ? 16 : 0;
    if (layout == RESKV_LAYOUT_COMPACT) return 16;
    return bits == 4 ? 8 : 16;  // structured INT4: two words; tiled / 4:16 FP16: four
}

unsigned char* at_token(void* base, int64_t token, size_t row_bytes) {
    return base ? static_cast<unsigned char*>(base) + static_cast<size_t>(token) * row_bytes : nullptr;
}

int pack_side(const Side& s, const int32_t* ids, int layout, int bits, int nnz, int batch, int kv_heads, int tokens,
              int64_t x_stride, int seq_len, void* stream) {
    void* payload = at_token(s.payload, seq_len, payload_row_bytes(layout, bits, nnz));
    void* meta = at_token(s.meta, seq_len, meta_row_bytes(layout, bits));
    void* scale = at_token(s.scale, seq_len, 2);
    const int c = s.new_clusters;
    if (layout == RESKV_LAYOUT_COMPACT)
        return reskv_encode_compact(s.x, s.new_centroids, ids, batch, kv_heads, tokens, x_stride, c, nnz, bits, payload,
                                    meta, scale, s.stride, stream);
    if (bits == 16 && layout == RESKV_LAYOUT_UNSTRUCTURED)
        return reskv_encode_bitmap_fp16(s.x, s.new_centroids, ids, batch, kv_heads, tokens, x_stride, c, nnz, payload,
                                        meta, s.stride, stream);
    if (bits == 16)
        return reskv_encode_tiled_fp16(s.x, s.new_centroids, ids, batch, kv_heads, tokens, x_stride, c, nnz,
                                       layout == RESKV_LAYOUT_STRUCTURED, payload, meta, s.stride, stream);
    if (layout == RESKV_LAYOUT_STRUCTURED)
        return reskv_encode_structured_int4(s.x, s.new_centroids, ids, batch, kv_heads, tokens, x_stride, c, payload,
                                            meta, scale, s.stride, stream);
    return reskv_encode_quantized(s.x, s.new_centroids, ids, batch, kv_heads, tokens, x_stride, c, nnz, bits, payload,
                                  scale, s.stride, stream);
}

}  // namespace
}  // namespace reskv

using namespace reskv;

extern "C" int reskv_compress_group(int layout, int bits, int nnz, const void* x_k, const void* x_v, int batch,
                                    int kv_heads, int tokens, int64_t x_tok_stride, const void* k_centroids_old,
                                    int k_clusters_old, void* k_centroids_new, int k_clusters_new, void* k_ids,
                                    void* k_payload, void* k_meta, void* k_scale, int64_t k_tok_stride,
                                    const void* v_centroids_old, int v_clusters_old, void* v_centroids_new,
                                    int v_clusters_new, void* v_ids, void* v_payload, void* v_meta, void* v_scale,
                                    int64_t v_tok_stride, int seq_len, int32_t* ids_scratch, void* stream) {
    if (!x_k || !x_v || !k_ids || !v_ids || !k_payload || !v_payload || !ids_scratch)
        return fail(RESKV_ERR_INVALID, "compress_group: null tensor pointer");
    if (batch < 1 || kv_heads < 1 || tokens < 1 || seq_len < 0)
        return fail(RESKV_ERR_INVALID, "compress_group: batch, heads and tokens must be positive, seq_len non-negative");
    if (static_cast<int64_t>(seq_len) + tokens > k_tok_stride || static_cast<int64_t>(seq_len) + tokens > v_tok_stride)
        return fail(RESKV_ERR_INVALID, "compress_group: %d + %d tokens do not fit the buffers (capacity %lld / %lld)",
                    seq_len, tokens, static_cast<long long>(k_tok_stride), static_cast<long long>(v_tok_stride));
    if (int rc = check_device_pointer(k_ids, "compress_group", "k_ids")) return rc;
    if (int rc = check_device_pointer(v_ids, "compress_group", "v_ids")) return rc;
    if (int rc = check_device_pointer(ids_scratch, "compress_group", "ids_scratch")) return rc;
    const Side sides[2] = {{x_k, k_centroids_old, k_clusters_old, k_centroids_new, k_clusters_new, k_ids, k_payload,
                            k_meta, k_scale, k_tok_stride},
                           {x_v, v_centroids_old, v_clusters_old, v_centroids_new, v_clusters_new, v_ids, v_payload,
                            v_meta, v_scale, v_tok_stride}};
    const int units = batch * kv_heads;
    int32_t* ids[2] = {ids_scratch, ids_scratch + static_cast<size_t>(units) * tokens};
    for (int i = 0; i < 2; ++i)
        if (int rc = reskv_kmeans_incremental(sides[i].x, batch, kv_heads, tokens, x_tok_stride, sides[i].old_centroids,
                                              sides[i].old_clusters, sides[i].new_centroids, sides[i].new_clusters,
                                              ids[i], stream))
            return rc;
    for (int i = 0; i < 2; ++i)
        if (int rc = pack_side(sides[i], ids[i], layout, bits, nnz, batch, kv_heads, tokens, x_tok_stride, seq_len, stream))
            return rc;
    const int total = units * tokens;
    narrow_ids_kernel<<<(total + kNarrowThreads - 1) / kNarrowThreads, kNarrowThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        ids[0], ids[1], static_cast<int8_t*>(k_ids) + seq_len, static_cast<int8_t*>(v_ids) + seq_len, tokens,
        k_tok_stride, v_tok_stride, total);
    return check_cuda(cudaGetLastError(), "compress_group: id rows launch");
}

extern "C" int reskv_window_shift(void* window_k, void* window_raw, void* window_v, int batch, int kv_heads,
                                  int window_capacity, int dst, int src, int count, void* stream) {
    if (!window_k || !window_raw || !window_v) return fail(RESKV_ERR_INVALID, "window_shift: null pointer");
    if (!aligned16(window_k) || !aligned16(window_raw) || !aligned16(window_v))
        return fail(RESKV_ERR_INVALID, "window_shift: buffers must be 16-byte aligned");
    if (batch < 1 || kv_heads < 1 || window_capacity < 1)
        return fail(RESKV_ERR_INVALID, "window_shift: batch, heads and capacity must be positive");
    if (dst < 0 || count < 0 || dst > src || static_cast<int64_t>(src) + count > window_capacity)
        return fail(RESKV_ERR_INVALID, "window_shift: need 0 <= dst <= src and src + count <= capacity");
    if (int rc = check_device_pointer(window_k, "window_shift", "window_k")) return rc;
    if (count == 0 || dst == src) return RESKV_OK;
    window_shift_kernel<<<dim3(batch * kv_heads, 3), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint4*>(window_k), static_cast<uint4*>(window_raw), static_cast<uint4*>(window_v), window_capacity,
        dst, src, count);
    return check_cuda(cudaGetLastError(), "window_shift launch");
}

/* C ABI of libreskv_b200.so: sm_100a kernels for the compressed-KV hot path.
 *
 * Every function takes plain device pointers, sizes and the CUDA stream to
 * launch on (a cudaStream_t passed as void*), never allocates device memory
 * unless it says so, never synchronises, and returns 0 on success or a
 * negative RESKV_ERR_* code; reskv_last_error() then describes the failure
 * (thread local).  Scratch memory is supplied by the caller: ask the matching
 * *_workspace_bytes() function for the size.
 *
 * Conventions shared by all entry points
 *   - head dimension is 128; B sequences, KH key/value heads, NH query heads;
 *     a "unit" is one (sequence, KV head) pair, unit = b * KH + h.
 *   - per-token tensors are addressed as base + (unit * tok_stride + t) * row,
 *     where tok_stride >= tokens is the capacity of the backing buffer in
 *     tokens (== tokens for plain contiguous tensors).
 *   - pointers to rows that are staged with bulk copies (bitmaps, payloads)
 *     must be 16-byte aligned.
 *
 * Each declaration cites the reference interface it replaces
 * (file:line within the coralabo/ResKV checkout).
 */
#ifndef RESKV_B200_H
#define RESKV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RESKV_OK 0
#define RESKV_ERR_INVALID (-1)   /* bad argument (shape, range, alignment, null pointer) */
#define RESKV_ERR_WORKSPACE (-2) /* workspace missing or too small */
#define RESKV_ERR_CUDA (-3)      /* a CUDA runtime call failed */
#define RESKV_ERR_LIMIT (-4)     /* size beyond a documented fixed maximum */

/* Bits of the 32-bit status word a kernel ORs into workspace[0] when something
 * went wrong on the device (read it after synchronising the stream). */
#define RESKV_STATUS_WAIT_TIMEOUT 1u /* a bounded wait on an async copy ran out */
#define RESKV_STATUS_STATE_RANGE 2u  /* a device-side count or slot index was out of range and got clamped / skipped */

/* Message of the last failure on the calling thread ("" if none). */
const char* reskv_last_error(void);

/* Library version, major * 10000 + minor * 100 + patch. */
int reskv_version(void);

/* ---- fused decode attention: unstructured FP16 bitmap layout ---------------
 *
 * Replaces cluster_mass.decode_fp16 (reskv/csrc/cluster_mass.cu:1177-1296, the
 * partial kernel :185-565 plus the split merge :1016-1104) and, when the
 * recent_* pointers are given, the recent-window merge that follows it
 * (reskv/_attention.py:117-143, cluster_mass.cu:1106-1169) in the same call.
 *
 *   q            f16 [B*NH,128]            query before RoPE
 *   k_centroids  f16 [B*KH,CK,128]         v_centroids f16 [B*KH,CV,128]
 *   k_ids/v_ids  i8  [B*KH,tok_stride]
 *   k_payload    f16 [B*KH,tok_stride,nnz] retained residuals, ascending coordinate
 *   k_bitmap     i64 [B*KH,tok_stride,2]   bit 63-d%64 of word d/64 marks coordinate d
 *   start_pos    position of compressed token 0;  pos_q  position of the query
 *   inv_freq     f32 [64] RoPE frequencies, or NULL for theta^(-i/64)
 *   splits       partitions of the token axis, 0 = choose from the SM count
 *   recent_q     f16 [B*NH,128] query after RoPE, recent_k (after RoPE) /
 *                recent_v f16 [B*KH,recent_tokens,128]; all NULL / 0 for none
 *   out          f16 [B*NH,128]
 *   out_m,out_l  f32 [B*NH] running maximum and un-normalised sum of the
 *                softmax over the compressed tokens only, or NULL
 */
size_t reskv_decode_bitmap_fp16_workspace_bytes(int batch, int kv_heads, int q_heads, int tokens, int splits);

int reskv_decode_bitmap_fp16(const void* q, const void* k_centroids, const void* k_ids, const void* k_payload,
                             const void* k_bitmap, const void* v_centroids, const void* v_ids,
                             const void* v_payload, const void* v_bitmap, int batch, int kv_heads, int q_heads,
                             int tokens, int64_t tok_stride, int k_clusters, int v_clusters, int nnz, int start_pos,
                             int pos_q, float rope_theta, const float* inv_freq, float scaling, int splits,
                             const void* recent_q, const void* recent_k, const void* recent_v, int recent_tokens,
                             void* workspace, size_t workspace_bytes, void* out, float* out_m, float* out_l,
                             void* stream);

/* ---- fused decode attention: the other residual layouts -----------------------------
 * Same contract as reskv_decode_bitmap_fp16 for
 *   RESKV_LAYOUT_UNSTRUCTURED, bits 4 / 2: payload i32 [.., 4*bits] (all 128 coords),
 *       no metadata, scale f16 [..] -- replaces attention.decode_quantized
 *       (reskv/csrc/attention.cu:967-1348);
 *   RESKV_LAYOUT_TILED, bits 16: payload f16 [.., 64], metadata i32 [.., 4] (16-bit
 *       tile masks) -- replaces attention.decode_fp16 (attention.cu:196-596,665-835);
 *   RESKV_LAYOUT_STRUCTURED, bits 16: payload f16 [.., 32], metadata i32 [.., 4]
 *       (4-bit in-tile indices) -- replaces attention.decode_fp16 and
 *       cluster_mass.decode_structured_fp16 (cluster_mass.cu:567-997,1298-1459);
 *   RESKV_LAYOUT_STRUCTURED, bits 4: payload i32 [.., 4], metadata i32 [.., 2], scale
 *       f16 [..] -- replaces attention.decode_int4 and
 *       cluster_mass.decode_structured_int4.
 * Per-token and deferred centroid fusion of the reference are the same sum; one
 * kernel serves both op families (value centroids are applied after the split
 * merge).  Workspace size as reskv_decode_bitmap_fp16_workspace_bytes. */
#define RESKV_LAYOUT_UNSTRUCTURED 0
#define RESKV_LAYOUT_TILED 1
#define RESKV_LAYOUT_STRUCTURED 2
#define RESKV_LAYOUT_COMPACT 3 /* reskv_decode_step only; see reskv_decode_compact */

int reskv_decode_packed(int layout, int bits, const void* q, const void* k_centroids, const void* k_ids,
                        const void* k_payload, const void* k_meta, const void* k_scale, const void* v_centroids,
                        const void* v_ids, const void* v_payload, const void* v_meta, const void* v_scale, int batch,
                        int kv_heads, int q_heads, int tokens, int64_t tok_stride, int k_clusters, int v_clusters,
                        int start_pos, int pos_q, float rope_theta, const float* inv_freq, float scaling, int splits,
                        const void* recent_q, const void* recent_k, const void* recent_v, int recent_tokens,
                        void* workspace, size_t workspace_bytes, void* out, float* out_m, float* out_l, void* stream);

/* ---- compact quantised residuals --------------------------------------------------------
 * No counterpart in the reference: its unstructured INT4 / INT2 layout stores all 128
 * coordinates of a token (discarded ones as 0).  The compact layout keeps the MSB-first
 * bitmap of the unstructured FP16 layout (i64 [.., 2]) and stores only the codes of the
 * nnz retained coordinates, in ascending coordinate order: words i32 [.., nnz*bits/32],
 * code of rank r at bit (r % (32/bits)) * bits of word r / (32/bits); scale f16 [..].
 * Selection, scale and codes are those of reskv_encode_quantized.  Supported: bits 4 with
 * nnz 64 or 32 (51 or 35 bytes per token and tensor instead of 67), bits 2 with nnz 64.
 * reskv_decode_compact takes the arguments of reskv_decode_packed with (bits, nnz) in
 * place of (layout, bits). */
int reskv_encode_compact(const void* x, const void* centroids, const int32_t* ids, int batch, int kv_heads, int tokens,
                         int64_t x_tok_stride, int clusters, int nnz, int bits, void* words, void* bitmap, void* scale,
                         int64_t out_tok_stride, void* stream);

int reskv_decode_compact(int bits, int nnz, const void* q, const void* k_centroids, const void* k_ids,
                         const void* k_payload, const void* k_bitmap, const void* k_scale, const void* v_centroids,
                         const void* v_ids, const void* v_payload, const void* v_bitmap, const void* v_scale, int batch,
                         int kv_heads, int q_heads, int tokens, int64_t tok_stride, int k_clusters, int v_clusters,
                         int start_pos, int pos_q, float rope_theta, const float* inv_freq, float scaling, int splits,
                         const void* recent_q, const void* recent_k, const void* recent_v, int recent_tokens,
                         void* workspace, size_t workspace_bytes, void* out, float* out_m, float* out_l, void* stream);

/* ---- decode steps that can be captured in a CUDA graph --------------------------------
 * No counterpart in the reference (its decode loop is eager Python,
 * benchmarks/timing.py:105-145, and passes positions by value).
 *
 * step_state is four int32 in device memory: {query position, tokens in the dense
 * window including the token of this step, compressed tokens or -1, reserved}.
 * reskv_window_append writes the new token's rotated key, raw key and value
 * (f16 [B*KH,128] each) into slot step_state[1] - 1 of the window buffers
 * (f16 [B*KH,window_capacity,128]); reskv_decode_step is reskv_decode_bitmap_fp16 /
 * reskv_decode_packed with the query position, the window length and -- when
 * step_state[2] >= 0 -- the compressed token count read from step_state inside the
 * kernels (layout UNSTRUCTURED with bits 16 selects the bitmap kernels, nnz = retained
 * coordinates per token, read for the bitmap and the compact layouts; `tokens` then only sizes the split count and is what the kernels use when
 * step_state[2] < 0; a count above tok_stride is cut to tok_stride; with 8-byte
 * metadata rows the count must keep the parity of `tokens`); reskv_step_advance adds
 * to the first two numbers.  A graph that holds "advance(0, 1), then per layer append +
 * decode, advance(1, 0)" can be replayed for consecutive steps.  It stays valid across
 * group compressions if the compressed segment grows in place (same addresses, token
 * stride and centroid-table shape: pass tables padded to a fixed number of rows, unused
 * rows finite) and the host writes the new counts into step_state between replays. */
int reskv_window_append(void* window_k, void* window_raw, void* window_v, const void* k_rot, const void* k_raw,
                        const void* v, int batch, int kv_heads, int window_capacity, const int32_t* step_state,
                        void* stream);

/* The same three-row copy for eager callers that track the window length on the host:
 * slot (0 <= slot < window_capacity) is given by value.  Replaces the three slice copies
 * of the reference's cache update (reskv/cache.py:55-60) by one launch. */
int reskv_window_write(void* window_k, void* window_raw, void* window_v, const void* k_rot, const void* k_raw,
                       const void* v, int batch, int kv_heads, int window_capacity, int slot, void* stream);

int reskv_decode_step(int layout, int bits, int nnz, const void* q, const void* k_centroids, const void* k_ids,
                      const void* k_payload, const void* k_meta, const void* k_scale, const void* v_centroids,
                      const void* v_ids, const void* v_payload, const void* v_meta, const void* v_scale, int batch,
                      int kv_heads, int q_heads, int tokens, int64_t tok_stride, int k_clusters, int v_clusters,
                      int start_pos, float rope_theta, const float* inv_freq, float scaling, int splits,
                      const void* recent_q, const void* window_k, const void* window_v, int window_capacity,
                      const int32_t* step_state, void* workspace, size_t workspace_bytes, void* out, void* stream);

int reskv_step_advance(int32_t* step_state, int position_increment, int window_increment, void* stream);

/* ---- the rest of a decoder layer's decode step, fused -----------------------------------
 * No counterpart in the reference (it runs Hugging Face modules, modeling.py); a decode
 * step at small batch is bound by launch count, and these replace ~30 tensor-op launches
 * per layer by three.  All tensors f16, row-major, on the device.
 *
 * reskv_rms_norm:   out[r] = x[r] * rsqrt(mean(x[r]^2) + eps) * weight, FP32 inside; dim % 8 == 0,
 *                   pointers 16-byte aligned.
 * reskv_rope_split: qkv [batch, (q_heads + 2 kv_heads) * 128] is the fused projection of one new
 *                   token per sequence, heads ordered q | k | v.  Writes the raw query (optional)
 *                   and the query rotated to position step_state[0] ([batch*q_heads,128] each);
 *                   the key rotated, the raw key and the value go to slot step_state[1] - 1 of
 *                   the window buffers ([batch*kv_heads,window_capacity,128]) when those are
 *                   given, and / or to k_rot / v_out ([batch*kv_heads,128]).
 * reskv_silu_mul:   out[r][j] = silu(gate_up[r][j]) * gate_up[r][ffn + j]; gate_up [rows, 2 ffn]. */
int reskv_rms_norm(const void* x, const void* weight, void* out, int rows, int dim, float eps, void* stream);

int reskv_rope_split(const void* qkv, int batch, int q_heads, int kv_heads, const float* inv_freq,
                     const int32_t* step_state, void* q_raw, void* q_rot, void* k_rot, void* v_out, void* window_k,
                     void* window_raw, void* window_v, int window_capacity, void* stream);

int reskv_silu_mul(const void* gate_up, void* out, int rows, int ffn, void* stream);

/* ---- decode attention for callers that cannot provide scratch memory -------------------
 * No counterpart in the reference (its ops allocate their partial buffers with
 * torch::empty on every call, cluster_mass.cu:1222-1232).
 *
 * Same computation, arguments and results as reskv_decode_bitmap_fp16, minus the
 * workspace: the split-K partials go to a fixed RESKV_NOALLOC_SCRATCH_BYTES array
 * that is part of the library image, so neither the caller nor the library calls
 * cudaMalloc / cudaFree (or any allocator) on this path.  It is meant for hosts
 * that have no allocator to offer at the call site: an inference server that gave
 * all device memory to its own pool at start-up, a plug-in invoked from a latency-
 * critical loop where an allocation would serialise the device, or a C / C++ /
 * cgo host that links the library without torch's caching allocator.
 *
 *   - Limit: batch * q_heads * slots * 776 + 256 bytes must fit the array (8 MiB:
 *     e.g. 1024 query heads x 10 slots), where slots = `splits` if given, else the
 *     library's own partial count (at most ceil(2 * SMs / (batch * kv_heads)) + 1).
 *     Larger problems are refused with RESKV_ERR_LIMIT and a message; pass a
 *     smaller `splits` or use the workspace variant.
 *   - Every GPU on which the library is loaded holds the array until exit.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress) and keeps it; make that first call outside any
 *     stream capture.  The kept address is written without a lock: two host
 *     threads making their first call on one device at the same time both look
 *     it up and store the same value.
 *   - All calls on a device share the array and it keeps the last call's contents;
 *     the call clears the 256-byte status header itself, after its arguments
 *     passed validation (a refused call writes nothing); read the status word
 *     with reskv_decode_noalloc_status.  Two calls whose kernels
 *     can overlap on the GPU (different streams, or graphs replayed concurrently)
 *     race on it: serialise them. */
#define RESKV_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024)

int reskv_decode_bitmap_fp16_noalloc(const void* q, const void* k_centroids, const void* k_ids,
                                     const void* k_payload, const void* k_bitmap, const void* v_centroids,
                                     const void* v_ids, const void* v_payload, const void* v_bitmap, int batch,
                                     int kv_heads, int q_heads, int tokens, int64_t tok_stride, int k_clusters,
                                     int v_clusters, int nnz, int start_pos, int pos_q, float rope_theta,
                                     const float* inv_freq, float scaling, int splits, const void* recent_q,
                                     const void* recent_k, const void* recent_v, int recent_tokens, void* out,
                                     float* out_m, float* out_l, void* stream);

/* The split count the fixed-split schedule would use for splits == 0 (what the warp-per-token kernel
 * runs with; the tensor-core kernel balances all tiles over two CTAs per SM instead, see
 * reskv_decode_bitmap_fp16_workspace_bytes for its scratch need). */
int reskv_decode_auto_splits(int batch, int kv_heads, int tokens);

/* Reads the device status word (RESKV_STATUS_* bits) that the kernels of reskv_decode_bitmap_fp16_noalloc
 * OR into the header of the built-in scratch: one 4-byte cudaMemcpyAsync to status_out (host memory;
 * pinned memory keeps the copy asynchronous) on `stream`, i.e. ordered behind the decode calls already
 * enqueued there.  Read status_out after synchronising the stream, and before the next noalloc call on
 * the device: that call clears the word.  No counterpart in the reference. */
int reskv_decode_noalloc_status(uint32_t* status_out, void* stream);

/* ---- recent-window merge ------------------------------------------------------
 * Replaces cluster_mass.merge_recent (cluster_mass.cu:1461-1508): joint softmax
 * of a finished compressed-attention result (out, m, l) with dense recent
 * tokens whose scaled scores [B*NH,recent_tokens] f32 the caller computed.
 * Writes merged f16 [B*NH,128]; may alias comp_out. */
int reskv_merge_recent_scores(const void* comp_out, const float* comp_m, const float* comp_l, const float* scores,
                              const void* recent_v, int batch, int kv_heads, int q_heads, int recent_tokens,
                              void* merged, void* stream);

/* Replaces attention.merge_recent (reskv/csrc/attention.cu:598-663,839-906):
 * same merge, scores computed here from the rotated query and rotated keys. */
int reskv_merge_recent_qk(const void* comp_out, const float* comp_m, const float* comp_l, const void* recent_q,
                          const void* recent_k, const void* recent_v, int batch, int kv_heads, int q_heads,
                          int recent_tokens, float scaling, void* merged, void* stream);

/* ---- residual packers ------------------------------------------------------------
 * Common arguments: x f16 [B*KH,x_tok_stride,128] (pre-RoPE K or V), centroids
 * f16 [B*KH,clusters,128], ids i32 [B*KH,tokens] (out-of-range ids are clamped,
 * like the reference kernels do; the Python layer validates them first).  Outputs
 * are addressed with out_tok_stride, so a group can be written straight behind
 * the live tokens of a capacity buffer.  r = fp32(x) - fp32(c); the selection key
 * is |fp16(r)|, larger first, lower coordinate on ties. */

/* Unstructured FP16: payload f16 [.., nnz] in ascending coordinate order, bitmap
 * i64 [.., 2] MSB first.  Replaces the torch path of _encode
 * (reskv/compression.py:75-89), which the reference runs as ~10 library kernels. */
int reskv_encode_bitmap_fp16(const void* x, const void* centroids, const int32_t* ids, int batch, int kv_heads,
                             int tokens, int64_t x_tok_stride, int clusters, int nnz, void* payload, void* bitmap,
                             int64_t out_tok_stride, void* stream);

/* Unstructured INT4 / INT2: words i32 [.., 4*bits] holding all 128 coordinates
 * (discarded ones 0), scale f16 [..].  Replaces compression.compress_quantized
 * (reskv/csrc/compression.cu:244-383,392-421). */
int reskv_encode_quantized(const void* x, const void* centroids, const int32_t* ids, int batch, int kv_heads,
                           int tokens, int64_t x_tok_stride, int clusters, int nnz, int bits, void* words,
                           void* scale, int64_t out_tok_stride, void* stream);

/* Tiled (structured == 0, 16-bit masks) or 4:16 structured (4-bit indices) FP16:
 * values f16 [.., nnz] in (tile, rank) order, meta i32 [.., 4].  x, centroids, values
 * and meta 16-byte aligned.  Replaces compression.compress_fp16
 * (reskv/csrc/compression.cu:57-147,423-473). */
int reskv_encode_tiled_fp16(const void* x, const void* centroids, const int32_t* ids, int batch, int kv_heads,
                            int tokens, int64_t x_tok_stride, int clusters, int nnz, int structured, void* values,
                            void* meta, int64_t out_tok_stride, void* stream);

/* 1-of-4 structured INT4: packed i32 [.., 4], meta i32 [.., 2], scale f16 [..].
 * x, centroids and packed 16-byte, meta 8-byte aligned.
 * Replaces compression.compress_structured_int4
 * (reskv/csrc/compression.cu:153-239,475-504). */
int reskv_encode_structured_int4(const void* x, const void* centroids, const int32_t* ids, int batch, int kv_heads,
                                 int tokens, int64_t x_tok_stride, int clusters, void* packed, void* meta,
                                 void* scale, int64_t out_tok_stride, void* stream);

/* ---- one decode group, appended in place ------------------------------------------------
 * What `compress(..., previous=cache)` does for the group that leaves the dense window
 * (reskv/compression.py:150-170 with _incremental_cluster :56-69 and _encode :72-101, then
 * CompressedTensor.append, reskv/tensors.py:105-119), for K and V in one call and without
 * intermediate tensors: reskv_kmeans_incremental of both sides, the packer of (layout, bits, nnz)
 * writing rows [seq_len, seq_len + tokens) of the cache's capacity buffers, the ids narrowed to
 * int8 into the same rows.  x_k / x_v f16 [B*KH,x_tok_stride,128]: the group's pre-RoPE keys and
 * its values (e.g. a token slice of the window buffers).  *_centroids_old f16
 * [B*KH,*_clusters_old,128], *_centroids_new [B*KH,*_clusters_new,128] with new == old or old + 1
 * (new may be the old table itself when the count stays).  *_ids int8 [B*KH,*_tok_stride];
 * *_payload / *_meta / *_scale: the buffers of the layout (null where it has none), every row
 * *_tok_stride tokens per unit, all given at token 0.  ids_scratch: int32 [2,B*KH,tokens].
 * Results are those of the separate calls, bit for bit. */
int reskv_compress_group(int layout, int bits, int nnz, const void* x_k, const void* x_v, int batch, int kv_heads,
                         int tokens, int64_t x_tok_stride, const void* k_centroids_old, int k_clusters_old,
                         void* k_centroids_new, int k_clusters_new, void* k_ids, void* k_payload, void* k_meta,
                         void* k_scale, int64_t k_tok_stride, const void* v_centroids_old, int v_clusters_old,
                         void* v_centroids_new, int v_clusters_new, void* v_ids, void* v_payload, void* v_meta,
                         void* v_scale, int64_t v_tok_stride, int seq_len, int32_t* ids_scratch, void* stream);

/* Moves tokens [src, src + count) of every unit of the three window buffers (f16
 * [B*KH,window_capacity,128], 16-byte aligned) to [dst, dst + count), dst <= src; the ranges may
 * overlap.  Replaces the slice copies that slide the window after a group left it
 * (reskv/cache.py:61-77). */
int reskv_window_shift(void* window_k, void* window_raw, void* window_v, int batch, int kv_heads, int window_capacity,
                       int dst, int src, int count, void* stream);

/* ---- clustering ------------------------------------------------------------------
 * Lloyd iterations per (sequence, KV head); replaces the torch loop of cluster()
 * (reskv/compression.py:19-53: cdist + argmin + one_hot + bmm per iteration).
 * Bit 0 of `value`: 0 = FP32 centres, empty clusters keep their centre (K); 1 =
 * centres rounded to FP16 each iteration, empty clusters become 0 (V).  Bit 1 of
 * `value`: accumulate the cluster sums as 2^24-scaled integers (every mean the
 * correctly rounded one) instead of the default for up to 32 centres, FP32 partial
 * sums formed on the tensor cores in a fixed order (same assignments, means within
 * one FP16 unit in the last place, several times faster; both forms are
 * reproducible).  That default runs on tcgen05.mma with TMA-fed token tiles (x must
 * be 16-byte aligned, otherwise the integer form is used); bit 2 of `value`
 * selects its earlier mma.sync form (kept as a cross-check for the tests).
 * Initial centres are the tokens at linspace(0, tokens-1, clusters).  Writes
 * centroids f16 [B*KH,clusters,128] (after the last update) and ids i32
 * [B*KH,tokens] (from the last assignment, i.e. relative to the centres before
 * that update -- the reference's loop order). */
size_t reskv_kmeans_workspace_bytes(int batch, int kv_heads, int clusters);

int reskv_kmeans(const void* x, int batch, int kv_heads, int tokens, int64_t x_tok_stride, int clusters,
                 int iterations, int value, void* workspace, size_t workspace_bytes, void* centroids, int32_t* ids,
                 void* stream);

/* Status word of the kernels of the last reskv_kmeans call on this workspace (RESKV_STATUS_* bits: a bounded
 * wait inside a kernel ran out; 0 = clean).  Copies 4 bytes to the host and synchronises `stream`. */
int reskv_kmeans_status(const void* workspace, int batch, int kv_heads, int clusters, uint32_t* status, void* stream);

/* Decode-time step; replaces _incremental_cluster (reskv/compression.py:56-69).
 * Copies old_centroids f16 [B*KH,old_clusters,128] into new_centroids
 * [B*KH,new_clusters,128]; when new_clusters == old_clusters + 1 the mean of the
 * group's tokens becomes the extra centre; then assigns the tokens to the
 * nearest centre. */
int reskv_kmeans_incremental(const void* x, int batch, int kv_heads, int tokens, int64_t x_tok_stride,
                             const void* old_centroids, int old_clusters, void* new_centroids, int new_clusters,
                             int32_t* ids, void* stream);

/* ---- test and profiling hooks ---------------------------------------------------------
 * NOT part of the surface a production host binds: both calls set process-wide state without any
 * synchronisation (they change what every thread's next decode call does) and exist for the test suite
 * (which runs every decode test on both partial kernels) and for bench.py (kernel time without launch
 * gaps).  No counterpart in the reference. */

/* Selects the partial kernel the decode entry points launch: 0 = tensor-core tiles of 16 tokens
 * (default), 1 = the simpler warp-per-token kernel (kept for cross-checking). */
int reskv_decode_set_variant(int variant);

/* cudaEvent_t handles that every following decode call records on its stream immediately before and
 * after the partial kernel.  NULL, NULL switches it off. */
int reskv_decode_set_timing_events(void* start, void* stop);

#ifdef __cplusplus
}
#endif
#endif /* RESKV_B200_H */

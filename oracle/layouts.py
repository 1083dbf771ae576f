"""Decoders of every residual bit layout (test infrastructure, numpy).

Restates ``reconstruct`` of the reference (reskv/reference.py:12-49).  A
compressed tensor is described here by plain arrays plus ``(layout, bits)``:

``centroids``  float16 ``[B,H,C,128]``
``ids``        integer ``[B,H,T]``
``payload``    float16 ``[B,H,T,nnz]`` or int32 words
``metadata``   int64 ``[B,H,T,2]`` / int32 ``[B,H,T,4|2]`` / ``None``
``scale``      float16 ``[B,H,T]`` / ``None``
"""

from __future__ import annotations

import numpy as np

HEAD_DIM = 128


def _u32(words: np.ndarray) -> np.ndarray:
    """int32 words reinterpreted as unsigned, widened so shifts stay logical."""
    return words.astype(np.int64) & 0xFFFFFFFF


def residual_unstructured_fp16(payload: np.ndarray, bitmap: np.ndarray) -> np.ndarray:
    """Bitmap layout (reference.py:21-26; written by compression.py:84-88).

    Coordinate ``d`` is kept when bit ``63 - d % 64`` of word ``d // 64`` is
    set; the payload lists kept coordinates in ascending ``d``.
    """
    dims = np.arange(HEAD_DIM)
    words = bitmap.astype(np.int64).view(np.uint64)[..., dims // 64]
    kept = ((words >> (63 - dims % 64).astype(np.uint64)) & np.uint64(1)).astype(bool)
    rank = np.cumsum(kept, axis=-1) - 1
    vals = np.take_along_axis(payload.astype(np.float32), np.clip(rank, 0, payload.shape[-1] - 1), axis=-1)
    return np.where(kept, vals, np.float32(0))


def mask_unstructured_fp16(bitmap: np.ndarray) -> np.ndarray:
    """Boolean ``[...,128]`` keep-mask stored in an MSB-first two-word bitmap."""
    dims = np.arange(HEAD_DIM)
    words = bitmap.astype(np.int64).view(np.uint64)[..., dims // 64]
    return ((words >> (63 - dims % 64).astype(np.uint64)) & np.uint64(1)).astype(bool)


def residual_quantized(words: np.ndarray, scale: np.ndarray, bits: int) -> np.ndarray:
    """Unstructured INT4 / INT2: all 128 coordinates, value ``i`` of a word at
    bit ``i * bits``, two's complement, times the token's FP16 scale
    (reference.py:16-20)."""
    per = 32 // bits
    shifts = np.arange(per) * bits
    q = (_u32(words)[..., None] >> shifts) & ((1 << bits) - 1)
    q = q.reshape(*words.shape[:-1], HEAD_DIM)
    sign = 1 << (bits - 1)
    q = (q ^ sign) - sign
    return q.astype(np.float32) * scale.astype(np.float32)[..., None]


def residual_compact(words: np.ndarray, bitmap: np.ndarray, scale: np.ndarray, bits: int) -> np.ndarray:
    """Compact quantised layout (no counterpart in the reference): the MSB-first
    bitmap of the unstructured FP16 layout says which coordinates are kept, the
    words hold the codes of the kept coordinates only, in ascending coordinate
    order, code ``i`` at bit ``(i % per) * bits`` of word ``i // per`` with
    ``per = 32 // bits``; codes and scale are those of the unstructured
    quantised layout."""
    per = 32 // bits
    shifts = np.arange(per) * bits
    q = (_u32(words)[..., None] >> shifts) & ((1 << bits) - 1)
    q = q.reshape(*words.shape[:-1], words.shape[-1] * per)
    sign = 1 << (bits - 1)
    q = ((q ^ sign) - sign).astype(np.float32)
    kept = mask_unstructured_fp16(bitmap)
    rank = np.cumsum(kept, axis=-1) - 1
    vals = np.take_along_axis(q, np.clip(rank, 0, q.shape[-1] - 1), axis=-1)
    return np.where(kept, vals, np.float32(0)) * scale.astype(np.float32)[..., None]


def residual_structured_int4(packed: np.ndarray, meta: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """1-of-4 INT4: 32 signed nibbles, 32 two-bit in-group indices
    (reference.py:27-36)."""
    q = (_u32(packed)[..., None] >> (np.arange(8) * 4)) & 15
    q = q.reshape(*packed.shape[:-1], 32)
    q = ((q ^ 8) - 8).astype(np.float32) * scale.astype(np.float32)[..., None]
    local = (_u32(meta)[..., None] >> (np.arange(16) * 2)) & 3
    dims = local.reshape(*meta.shape[:-1], 32) + np.arange(32) * 4
    out = np.zeros((*packed.shape[:-1], HEAD_DIM), np.float32)
    np.put_along_axis(out, dims, q, axis=-1)
    return out


def _tile_codes(meta: np.ndarray) -> np.ndarray:
    """Eight 16-bit per-tile codes from four int32 words (low half first)."""
    w = _u32(meta)
    return np.stack((w & 0xFFFF, (w >> 16) & 0xFFFF), axis=-1).reshape(*meta.shape[:-1], 8)


def residual_structured_fp16(payload: np.ndarray, meta: np.ndarray) -> np.ndarray:
    """4:16 FP16: per 16-wide tile four 4-bit in-tile indices, payload in
    (tile, rank) order (reference.py:37-43)."""
    codes = _tile_codes(meta)
    dims = ((codes[..., None] >> (np.arange(4) * 4)) & 15) + (np.arange(8) * 16)[:, None]
    out = np.zeros((*payload.shape[:-1], HEAD_DIM), np.float32)
    np.put_along_axis(out, dims.reshape(*payload.shape[:-1], 32), payload.astype(np.float32), axis=-1)
    return out


def residual_tiled_fp16(payload: np.ndarray, meta: np.ndarray) -> np.ndarray:
    """Tiled FP16: one 16-bit LSB-first mask per tile, payload in ascending
    coordinate order (reference.py:44-48)."""
    codes = _tile_codes(meta)
    kept = ((codes[..., None] >> np.arange(16)) & 1).astype(bool).reshape(*payload.shape[:-1], HEAD_DIM)
    rank = np.cumsum(kept, axis=-1) - 1
    vals = np.take_along_axis(payload.astype(np.float32), np.clip(rank, 0, payload.shape[-1] - 1), axis=-1)
    return np.where(kept, vals, np.float32(0))


def residual(layout: str, bits: int, payload, metadata, scale) -> np.ndarray:
    """Dense float32 residual ``[B,H,T,128]`` of any layout."""
    if layout == "compact":
        return residual_compact(payload, metadata, scale, bits)
    if layout == "unstructured" and bits != 16:
        return residual_quantized(payload, scale, bits)
    if layout == "unstructured":
        return residual_unstructured_fp16(payload, metadata)
    if bits == 4:
        return residual_structured_int4(payload, metadata, scale)
    if layout == "structured":
        return residual_structured_fp16(payload, metadata)
    if layout == "tiled":
        return residual_tiled_fp16(payload, metadata)
    raise ValueError(f"unknown layout {layout!r}")


def reconstruct(layout: str, bits: int, centroids, ids, payload, metadata=None, scale=None) -> np.ndarray:
    """Dense float32 ``[B,H,T,128]``: centroid of each token plus its residual
    (reference.py:12-49)."""
    idx = np.broadcast_to(ids.astype(np.int64)[..., None], (*ids.shape, HEAD_DIM))
    centres = np.take_along_axis(centroids.astype(np.float32), idx, axis=2)
    return centres + residual(layout, bits, payload, metadata, scale)

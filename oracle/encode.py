"""Residual packers (test infrastructure, numpy).

Restates the four encoders of the reference:

* unstructured FP16 bitmap -- ``_encode`` in reskv/compression.py:75-89 (torch
  ops; its tie order among equal magnitudes is whatever ``topk`` / ``sort``
  return, so the rule of the reference's own CUDA packers is fixed here:
  larger ``|fp16(r)|`` first, lower coordinate on ties);
* tiled / 4:16 structured FP16 -- reskv/csrc/compression.cu:57-147;
* 1-of-4 structured INT4 -- reskv/csrc/compression.cu:153-239;
* unstructured INT4 / INT2 -- reskv/csrc/compression.cu:244-383.

All take ``x`` float16 ``[B,H,T,128]``, ``centroids`` float16 ``[B,H,C,128]``,
``ids`` integer ``[B,H,T]``.  Rounding points: ``r = fp32(x) - fp32(c)``; the
selection key is ``|fp16(r)|``; FP16 layouts store ``fp16(r)``; quantisers
divide the FP32 ``r``.
"""

from __future__ import annotations

import numpy as np

HEAD_DIM = 128


def residual_fp32(x: np.ndarray, centroids: np.ndarray, ids: np.ndarray) -> np.ndarray:
    """``fp32(x) - fp32(centroid[id])`` (compression.cu:86-90; out-of-range ids
    are clamped there, callers validate instead)."""
    idx = np.broadcast_to(ids.astype(np.int64)[..., None], (*ids.shape, HEAD_DIM))
    c = np.take_along_axis(centroids.astype(np.float32), idx, axis=2)
    return x.astype(np.float32) - c


def _keys(r32: np.ndarray) -> np.ndarray:
    """Selection key ``|fp16(r)|`` as float32 (compression.cu:92-93)."""
    return np.abs(r32.astype(np.float16)).astype(np.float32)


def topk_mask(keys: np.ndarray, k: int) -> np.ndarray:
    """Boolean mask of the ``k`` largest keys along the last axis, lower index
    winning ties (compression.cu:109, :304-305)."""
    order = np.argsort(-keys, axis=-1, kind="stable")[..., :k]
    mask = np.zeros(keys.shape, bool)
    np.put_along_axis(mask, order, True, axis=-1)
    return mask


def tie_tokens(keys: np.ndarray, k: int) -> np.ndarray:
    """Tokens whose ``k``-th and ``k+1``-th largest keys are equal: there the
    reference's torch path (compression.py:79-83) may keep either coordinate."""
    s = -np.sort(-keys, axis=-1)
    return s[..., k - 1] == s[..., k]


def encode_unstructured_fp16(x, centroids, ids, nnz: int):
    """-> ``(payload f16 [B,H,T,nnz], bitmap i64 [B,H,T,2])``.

    Bit ``63 - d % 64`` of word ``d // 64`` marks coordinate ``d``
    (compression.py:84-88); payload in ascending ``d``.
    """
    r32 = residual_fp32(x, centroids, ids)
    r16 = r32.astype(np.float16)
    mask = topk_mask(_keys(r32), nnz)
    order = np.argsort(~mask, axis=-1, kind="stable")[..., :nnz]  # kept dims, ascending
    payload = np.take_along_axis(r16, order, axis=-1)
    weights = np.uint64(1) << np.arange(63, -1, -1, dtype=np.uint64)
    words = (mask.reshape(*mask.shape[:-1], 2, 64).astype(np.uint64) * weights).sum(-1, dtype=np.uint64)
    return payload, words.view(np.int64)


def _tile_masks(keys: np.ndarray, per_tile: int) -> np.ndarray:
    """Top ``per_tile`` of every 16-wide tile -> bool ``[...,8,16]``."""
    return topk_mask(keys.reshape(*keys.shape[:-1], 8, 16), per_tile)


def encode_tiled_fp16(x, centroids, ids, nnz: int, structured: bool):
    """-> ``(values f16 [B,H,T,nnz], meta i32 [B,H,T,4])`` (compression.cu:57-147).

    ``nnz // 8`` coordinates per tile; values in (tile, ascending coordinate)
    order.  ``meta`` word ``w`` carries tile ``2w`` in its low and tile ``2w+1``
    in its high 16 bits: an LSB-first mask, or -- ``structured`` -- four 4-bit
    in-tile indices, rank ``r`` at bit ``4r`` (compression.cu:44-55,128-136).
    """
    r32 = residual_fp32(x, centroids, ids)
    r16 = r32.astype(np.float16)
    masks = _tile_masks(_keys(r32), nnz // 8)
    flat = masks.reshape(*masks.shape[:-2], HEAD_DIM)
    order = np.argsort(~flat, axis=-1, kind="stable")[..., :nnz]
    values = np.take_along_axis(r16, order, axis=-1)
    if structured:
        local = (order % 16).reshape(*order.shape[:-1], 8, 4).astype(np.int64)
        codes = (local << (np.arange(4) * 4)).sum(-1)
    else:
        codes = (masks.astype(np.int64) << np.arange(16)).sum(-1)
    words = codes[..., 0::2] | (codes[..., 1::2] << 16)
    return values, words.astype(np.uint32).view(np.int32)


def near_half_integer(quotient: np.ndarray, ulps: int = 4) -> np.ndarray:
    """Quotients within ``ulps`` float32 units in the last place of ``n + 1/2``.

    The reference is built with ``--use_fast_math``, so its divisions are the GPU's approximate
    ``div.approx.ftz.f32`` (a reciprocal of up to 1 ulp error times the numerator) where this restatement
    divides exactly.  The two can round to different integers only when the quotient sits this close to a
    rounding boundary; the CUDA kernels of this repository issue the same approximate division as the
    reference, the comparisons against *this* restatement set those codes aside and count them."""
    q = np.abs(quotient.astype(np.float64))
    dist = np.abs(q - (np.floor(q) + 0.5))
    return dist <= ulps * np.spacing(np.maximum(q, 1.0).astype(np.float32)).astype(np.float64)


def encode_structured_int4(x, centroids, ids, return_ambiguous: bool = False):
    """-> ``(packed i32 [B,H,T,4], meta i32 [B,H,T,2], scale f16 [B,H,T])``.

    One coordinate of every four (compression.cu:189-204), scale
    ``s = amax * fp32(1/7)`` kept in FP32 for the division and stored as FP16
    (:224-227), ``q = clamp(rint(r / s), -7, 7)`` (:233-235).  With
    ``return_ambiguous`` a fourth result marks the groups ``[B,H,T,32]`` whose
    quotient lies on a rounding boundary (see ``near_half_integer``).
    """
    r32 = residual_fp32(x, centroids, ids)
    groups = _keys(r32).reshape(*r32.shape[:-1], 32, 4)
    best = np.argmax(groups, axis=-1)  # first maximum = lower index on ties
    compact = np.take_along_axis(r32.reshape(*r32.shape[:-1], 32, 4), best[..., None], axis=-1)[..., 0]
    amax = np.abs(compact).max(-1)
    s = np.where(amax > 0, amax * (np.float32(1.0) / np.float32(7.0)), np.float32(1.0)).astype(np.float32)
    quotient = compact / s[..., None]
    q = np.clip(np.rint(quotient), -7, 7).astype(np.int64) & 15
    packed = (q.reshape(*q.shape[:-1], 4, 8) << (np.arange(8) * 4)).sum(-1)
    meta = (best.astype(np.int64).reshape(*best.shape[:-1], 2, 16) << (np.arange(16) * 2)).sum(-1)
    out = (packed.astype(np.uint32).view(np.int32), meta.astype(np.uint32).view(np.int32), s.astype(np.float16))
    return (*out, near_half_integer(quotient)) if return_ambiguous else out


def quantized_codes(r32: np.ndarray, mask: np.ndarray, bits: int):
    """Scale and signed codes of the unstructured quantiser -> ``(h f16 [...], q int64 [...,128],
    quotient f32 [...,128])`` (compression.cu:354-368).

    ``h = fp16(amax * fp32(1 / QMAX))``: the reference divides by the constant ``QMAX`` under
    ``--use_fast_math``, which the compiler turns into a multiplication by the rounded reciprocal (pinned by a
    recorded token whose two forms round to different FP16 values).  ``q = clamp(lrintf(r / fp32(h)))`` for
    kept coordinates, 0 for discarded ones.  When ``h`` underflows to 0 (all kept residuals below
    ``QMAX * 2**-25``) the quotient is +-inf or NaN and the reference's ``(int)lrintf(.)`` keeps the low 32 bits
    of the saturated 64-bit conversion: -1 for positive residuals, 0 for negative ones and for zeros.
    """
    qmax = (1 << (bits - 1)) - 1
    amax = np.where(mask, np.abs(r32), np.float32(0)).max(-1).astype(np.float32)
    recip = np.float32(1.0) / np.float32(qmax)
    h = np.where(amax > 0, amax * recip, np.float32(1.0)).astype(np.float32).astype(np.float16)
    hf = h.astype(np.float32)[..., None]
    with np.errstate(divide="ignore", invalid="ignore"):
        quotient = (r32 / hf).astype(np.float32)
        q = np.clip(np.rint(quotient), -qmax, qmax)
    q = np.where(hf == 0, np.where(r32 > 0, -1.0, 0.0), np.nan_to_num(q))
    return h, np.where(mask, q, 0).astype(np.int64), np.where(mask & (hf != 0), quotient, np.float32(0))


def encode_quantized(x, centroids, ids, nnz: int, bits: int, return_ambiguous: bool = False):
    """-> ``(words i32 [B,H,T,4*bits], scale f16 [B,H,T])`` (compression.cu:244-383).

    Global top-``nnz`` of 128; scale and codes as in ``quantized_codes``; every coordinate
    is stored, discarded ones as 0; value ``i`` of a word at bit ``i * bits``.  With
    ``return_ambiguous`` a third result marks the coordinates ``[B,H,T,128]`` whose
    quotient lies on a rounding boundary (see ``near_half_integer``).
    """
    r32 = residual_fp32(x, centroids, ids)
    mask = topk_mask(_keys(r32), nnz)
    h, q, quotient = quantized_codes(r32, mask, bits)
    q = q & ((1 << bits) - 1)
    per = 32 // bits
    words = (q.reshape(*q.shape[:-1], HEAD_DIM // per, per) << (np.arange(per) * bits)).sum(-1)
    out = (words.astype(np.uint32).view(np.int32), h)
    return (*out, near_half_integer(quotient) & mask) if return_ambiguous else out


def encode_compact(x, centroids, ids, nnz: int, bits: int):
    """-> ``(words i32 [B,H,T,nnz*bits/32], bitmap i64 [B,H,T,2], scale f16 [B,H,T])``.

    Same selection, scale and codes as ``encode_quantized``; only the kept
    coordinates are stored (ascending coordinate order) next to the MSB-first
    bitmap of the unstructured FP16 layout.  No counterpart in the reference.
    """
    r32 = residual_fp32(x, centroids, ids)
    mask = topk_mask(_keys(r32), nnz)
    h, q, _ = quantized_codes(r32, mask, bits)
    q = q & ((1 << bits) - 1)
    order = np.argsort(~mask, axis=-1, kind="stable")[..., :nnz]  # kept coordinates, ascending
    codes = np.take_along_axis(q, order, axis=-1)
    per = 32 // bits
    words = (codes.reshape(*codes.shape[:-1], nnz // per, per) << (np.arange(per) * bits)).sum(-1)
    weights = np.uint64(1) << (np.uint64(63) - np.arange(64, dtype=np.uint64))
    bitmap = (mask.reshape(*mask.shape[:-1], 2, 64).astype(np.uint64) * weights).sum(-1, dtype=np.uint64)
    return words.astype(np.uint32).view(np.int32), bitmap.view(np.int64), h


def encode(layout: str, bits: int, nnz: int, x, centroids, ids):
    """Dispatch by plan -> ``(payload, metadata or None, scale or None)``
    (compression.py:72-101)."""
    if layout == "compact":
        return encode_compact(x, centroids, ids, nnz, bits)
    if bits == 16 and layout == "unstructured":
        p, m = encode_unstructured_fp16(x, centroids, ids, nnz)
        return p, m, None
    if bits == 16:
        p, m = encode_tiled_fp16(x, centroids, ids, nnz, layout == "structured")
        return p, m, None
    if layout == "structured":
        return encode_structured_int4(x, centroids, ids)
    p, s = encode_quantized(x, centroids, ids, nnz, bits)
    return p, None, s

"""FP32 decode attention over a reconstructed cache (test infrastructure, numpy).

Restates ``rotate`` and ``reference_attention`` of the reference
(reskv/reference.py:52-91): half-split RoPE (coordinate ``i`` pairs with
``i + 64``, frequency index ``i``), keys rotated at ``start_position + t``, the
query at ``position``, one softmax over compressed and recent tokens together.
"""

from __future__ import annotations

import numpy as np

from . import layouts


def theta_frequencies(rope_theta: float) -> np.ndarray:
    """``theta ** (-i / 64)`` for ``i < 64`` in float32 (reference.py:73-77)."""
    return (np.float32(rope_theta) ** (-(np.arange(64, dtype=np.float32) / np.float32(64)))).astype(np.float32)


def rotate(x: np.ndarray, positions: np.ndarray, frequencies: np.ndarray) -> np.ndarray:
    """Rotate ``x [...,P,128]`` at ``positions [P]`` (reference.py:52-56).
    The angle is formed in float32 like the reference's."""
    ang = positions.astype(np.float32)[:, None] * frequencies.astype(np.float32)[None, :]
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    a, b = x.astype(np.float32)[..., :64], x.astype(np.float32)[..., 64:]
    return np.concatenate((a * cos - b * sin, b * cos + a * sin), axis=-1)


def attention_dense(
    query: np.ndarray,
    keys: np.ndarray,
    values: np.ndarray,
    *,
    position: int,
    start_position: int = 0,
    rope_theta: float = 500000.0,
    inv_freq: np.ndarray | None = None,
    scaling: float | None = None,
    recent: tuple | None = None,
    return_stats: bool = False,
):
    """Attention of ``query [B,nh,1,128]`` (pre-RoPE) over pre-RoPE ``keys`` /
    ``values`` ``[B,kh,T,128]`` plus optional ``recent = (rotated q, rotated k,
    v)``.  -> float32 ``[B,nh,1,128]`` (reference.py:69-91).

    With ``return_stats`` also the running maximum and un-normalised sum of the
    softmax over the *compressed* tokens only, the two numbers the decode
    kernels hand to the recent-window merge.
    """
    b, kh, t, _ = keys.shape
    nh = query.shape[1]
    g = nh // kh
    freq = theta_frequencies(rope_theta) if inv_freq is None else inv_freq.astype(np.float32)
    # query heads of one KV head are batched as rows [B,kh,g,128] instead of
    # repeating K and V g times (reference.py:80); the arithmetic is the same
    q = rotate(query, np.array([position]), freq).reshape(b, kh, g, 128)
    k = rotate(keys, np.arange(start_position, start_position + t), freq)
    v = values.astype(np.float32)
    scale = np.float32(128**-0.5 if scaling is None else scaling)
    scores = np.matmul(q, k.transpose(0, 1, 3, 2)) * scale  # [B,kh,g,T]
    stats = None
    if return_stats:
        m = scores.max(-1)
        stats = (m.reshape(b, nh), np.exp(scores - m[..., None]).sum(-1).reshape(b, nh))
    if recent is not None and recent[1].shape[2] > 0:
        qr, kr, vr = recent
        qr = qr.astype(np.float32).reshape(b, kh, g, 128)
        rs = np.matmul(qr, kr.astype(np.float32).transpose(0, 1, 3, 2)) * scale
        scores = np.concatenate((scores, rs), axis=-1)
        v = np.concatenate((v, vr.astype(np.float32)), axis=2)
    scores = scores - scores.max(-1, keepdims=True)
    p = np.exp(scores)
    p = p / p.sum(-1, keepdims=True)
    out = np.matmul(p, v).astype(np.float32).reshape(b, nh, 1, 128)
    return (out, *stats) if return_stats else out


def attention_compressed(query, key_cache: dict, value_cache: dict, **kw):
    """``reference_attention`` on compressed caches given as dicts with keys
    ``layout, bits, centroids, ids, payload, metadata, scale``."""
    k = layouts.reconstruct(**key_cache)
    v = layouts.reconstruct(**value_cache)
    return attention_dense(query, k, v, **kw)

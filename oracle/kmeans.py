"""Lloyd clustering per (sequence, KV head) (test infrastructure, numpy).

Restates ``cluster`` (reskv/compression.py:19-53) and ``_incremental_cluster``
(reskv/compression.py:56-69).

What the reference leaves to libraries is fixed here as follows.  Distances in
the reference come from ``torch.cdist`` (matrix-multiply form, FP16 for V),
whose rounding decides near-ties arbitrarily; the contract restated here is the
*exact* nearest centre -- squared distances accumulated in float64 -- with the
lowest index on ties.  ``margin`` (gap between the two smallest squared
distances, relative) is returned so that a comparison can set aside tokens
whose choice no float32 evaluation can be expected to reproduce.
"""

from __future__ import annotations

import numpy as np


def init_indices(t: int, count: int) -> np.ndarray:
    """Token indices of the initial centres: ``linspace(0, t-1, count).long()``
    (compression.py:35).  torch evaluates linspace in float32, symmetric about
    the midpoint, and truncates."""
    if count == 1:
        return np.zeros(1, np.int64)
    step = np.float32(np.float32(t - 1) / np.float32(count - 1))
    i = np.arange(count)
    # torch forms both halves with a fused multiply-add: the product is exact
    # (float64 holds it), one rounding to float32 at the end.
    lo = (np.float64(step) * i).astype(np.float32)
    hi = (np.float64(t - 1) - np.float64(step) * (count - 1 - i)).astype(np.float32)
    return np.where(i < count // 2, lo, hi).astype(np.int64)


def assign(data: np.ndarray, centres: np.ndarray):
    """Nearest centre per token.

    data ``[N,T,128]``, centres ``[N,C,128]`` (any float dtype; values are used
    as given) -> ``(ids int32 [N,T], margin float64 [N,T])``.
    """
    x = data.astype(np.float64)
    c = centres.astype(np.float64)
    # |x-c|^2 up to the per-token constant |x|^2
    d = (c * c).sum(-1)[:, None, :] - 2.0 * np.einsum("ntd,ncd->ntc", x, c)
    ids = d.argmin(-1)
    if c.shape[1] > 1:
        part = np.partition(d, 1, axis=-1)
        full = part[..., 0] + (x * x).sum(-1)
        margin = (part[..., 1] - part[..., 0]) / np.maximum(np.abs(full), 1e-30)
    else:
        margin = np.full(ids.shape, np.inf)
    return ids.astype(np.int32), margin


def update(data: np.ndarray, ids: np.ndarray, centres: np.ndarray, value: bool) -> np.ndarray:
    """One centre update (compression.py:40-52).

    K (``value=False``): float32 mean, an empty cluster keeps its centre.
    V: float32-accumulated mean rounded to float16, an empty cluster becomes 0.
    """
    n, t, dim = data.shape
    count = centres.shape[1]
    sums = np.zeros((n, count, dim), np.float64)
    counts = np.zeros((n, count), np.float64)
    for u in range(n):
        np.add.at(sums[u], ids[u], data[u].astype(np.float64))
        counts[u] = np.bincount(ids[u], minlength=count)
    mean = (sums / np.maximum(counts, 1)[..., None]).astype(np.float32)
    if value:
        return mean.astype(np.float16)
    return np.where(counts[..., None] > 0, mean, centres.astype(np.float32))


def cluster(x: np.ndarray, count: int = 32, iterations: int = 10, value: bool = False):
    """-> ``(centres f16 [B,H,C,128], ids i32 [B,H,T], margin)``.

    Follows compression.py:19-53 including its loop order: the returned ids are
    those of the *last assignment*, i.e. relative to the centres before the
    final update.  ``t < count`` (jittered extra centres drawn from the global
    RNG, :28-33) is only reproduced for V, where ``count`` is clamped to ``t``.
    """
    b, h, t, dim = x.shape
    count = min(count, t) if value else count
    if t < count:
        raise ValueError("oracle does not restate the randomly jittered short-input initialisation")
    data = x.reshape(b * h, t, dim)
    data = data.astype(np.float16) if value else data.astype(np.float32)
    centres = data[:, init_indices(t, count)].copy()
    ids = margin = None
    for _ in range(iterations):
        ids, margin = assign(data, centres)
        centres = update(data, ids, centres, value)
    return (
        centres.astype(np.float16).reshape(b, h, count, dim),
        ids.reshape(b, h, t),
        margin.reshape(b, h, t),
    )


def incremental(x: np.ndarray, centres: np.ndarray, max_clusters: int, value: bool = False):
    """Decode-time step (compression.py:56-69): while below ``max_clusters``
    append the group mean (in ``x``'s dtype, float16) as a new centre, then
    assign the group's tokens.  -> ``(centres f16, ids i32, margin)``."""
    b, h, t, dim = x.shape
    if centres.shape[2] < max_clusters:
        mean = x.astype(np.float32).mean(2, keepdims=True).astype(np.float16)
        centres = np.concatenate((centres.astype(np.float16), mean), axis=2)
    ids, margin = assign(x.reshape(b * h, t, dim), centres.reshape(b * h, -1, dim))
    return centres, ids.reshape(b, h, t), margin.reshape(b, h, t)

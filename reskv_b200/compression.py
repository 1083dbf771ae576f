"""Clustering and residual compression of pre-RoPE K and V.

Public surface of the reference module (reskv/compression.py): ``cluster``,
``compress``, and the internal ``_incremental_cluster`` / ``_encode`` that
``compress`` is made of.  Every numeric step is a kernel of the native library;
this file only validates, allocates and wires results into ``CompressedTensor``.
"""

from __future__ import annotations

import torch

from ._extension import load_extension
from .config import KernelPlan, ResKVKernelConfig
from .tensors import CompressedKV, CompressedTensor

_INT_DTYPES = (torch.int8, torch.int16, torch.int32, torch.int64)


def _validate(x: torch.Tensor):
    if x.ndim != 4 or x.shape[-1] != 128 or not x.is_cuda or x.dtype != torch.float16:
        raise ValueError("expected FP16 CUDA tensor [batch, kv_heads, tokens, 128]")
    if min(x.shape[:3]) < 1:
        raise ValueError("batch, head and token dimensions must be nonempty")


def _ops(x: torch.Tensor):
    return load_extension("compression", device_index=x.device.index or 0)


@torch.no_grad()
def cluster(x: torch.Tensor, count: int = 32, iterations: int = 10, *, value: bool = False):
    """Lloyd clustering per (sequence, KV head) -> ``(centres f16 [B,H,C,128],
    ids i32 [B,H,T])`` (reference compression.py:19-53).

    K (``value=False``) iterates FP32 centres and keeps the centre of an empty
    cluster; V rounds centres to FP16 every iteration and zeroes empty ones.
    Initial centres are the tokens at ``linspace(0, T-1, C)``.  As in the
    reference the returned ids belong to the last assignment step, i.e. to the
    centres *before* the final update.

    Differences, both in what the reference leaves to libraries: assignments are
    the exact nearest centre with the lowest index on ties (the reference takes
    whatever ``torch.cdist``'s matrix form rounds to, in FP16 for V), and for
    ``T < count`` on the K path the surplus centres repeat tokens instead of
    adding jitter from the global RNG.
    """
    _validate(x)
    t = x.shape[2]
    if value:
        count = min(count, t)
    return _ops(x).kmeans(x.contiguous(), int(count), int(iterations), value)


@torch.no_grad()
def _incremental_cluster(x, centers, config, *, value=False):
    """Append the group mean as a new centre until the limit is reached, then
    assign the group's tokens (reference compression.py:56-69)."""
    append = centers.shape[2] < config.max_clusters
    return _ops(x).kmeans_incremental(x.contiguous(), centers.half(), append)


@torch.no_grad()
def _encode(x, centers, ids, plan: KernelPlan, *, value=False):
    """Residuals of ``x`` to its centres in the layout of ``plan``
    (reference compression.py:72-101).  ``value`` is accepted for signature
    compatibility: K and V use the same selection rule here."""
    ids = ids.int().contiguous()
    centers = centers.half().contiguous()
    x = x.contiguous()
    ops = _ops(x)
    metadata = scale = None
    if plan.layout == "compact":
        payload, metadata, scale = ops.compress_compact(x, centers, ids, plan.nnz, plan.bits)
    elif plan.bits == 16 and plan.layout == "unstructured":
        payload, metadata = ops.compress_bitmap_fp16(x, centers, ids, plan.nnz)
    elif plan.bits == 16:
        payload, metadata = ops.compress_fp16(x, centers, ids, plan.nnz, plan.layout == "structured")
    elif plan.layout == "structured":
        payload, metadata, scale = ops.compress_structured_int4(x, centers, ids)
    else:
        payload, scale = ops.compress_quantized(x, centers, ids, plan.nnz, plan.bits)
    return CompressedTensor(centers, ids, payload, metadata, scale, plan)


@torch.no_grad()
def compress(
    key: torch.Tensor,
    value: torch.Tensor,
    config: ResKVKernelConfig | None = None,
    *,
    previous: CompressedKV | None = None,
    clustering: tuple | None = None,
    plan: KernelPlan | None = None,
) -> CompressedKV:
    """Compress pre-RoPE K and unrotated V; optionally append a decode group.

    Same contract as the reference (compression.py:104-170):
    ``clustering=((k_centres, k_ids), (v_centres, v_ids))`` injects external
    clustering, ``previous`` extends an existing cache (its centroid tables grow
    by one group mean until ``config.max_clusters``).
    """
    config = ResKVKernelConfig() if config is None else config
    if not isinstance(config, ResKVKernelConfig):
        raise TypeError("compress requires ResKVKernelConfig; ResKVConfig is for accuracy evaluation")
    _validate(key)
    _validate(value)
    if key.shape != value.shape or key.device != value.device:
        raise ValueError("K and V must have identical shapes and devices")
    plan = plan or (previous.key.plan if previous else config.resolve(key.shape[0]))
    if plan.bits != config.bits or plan.nnz != int(128 * config.keep_ratio):
        raise ValueError("compression plan and configuration disagree")
    if config.layout != "auto" and plan.layout != config.layout:
        raise ValueError("compression plan violates the requested layout")
    if config.centroid_fusion != "auto" and plan.centroid_fusion != config.centroid_fusion:
        raise ValueError("compression plan violates the requested centroid fusion")
    if plan.fixed_shift != (config.softmax_mode == "fixed_shift"):
        raise ValueError("compression plan and softmax configuration disagree")
    if previous is not None:
        pk = previous.key
        if pk.cluster_ids.shape[:2] != key.shape[:2] or pk.centroids.device != key.device:
            raise ValueError("previous cache has incompatible dimensions or device")
        if max(pk.centroids.shape[2], previous.value.centroids.shape[2]) > config.max_clusters:
            raise ValueError("previous cache exceeds the configured centroid limit")
    if clustering is not None and previous is not None:
        raise ValueError("provide clustering or previous, not both")
    if clustering is not None:
        (kc, ki), (vc, vi) = clustering
        for centers, ids in ((kc, ki), (vc, vi)):
            if centers.ndim != 4 or centers.shape[:2] != key.shape[:2] or centers.shape[-1] != 128:
                raise ValueError("external centers must have shape [B,H,C,128]")
            if not 1 <= centers.shape[2] <= config.max_clusters or ids.shape != key.shape[:3]:
                raise ValueError("external clustering has incompatible sizes")
            if centers.device != key.device or ids.device != key.device:
                raise ValueError("external clustering must share the K/V device")
            if ids.dtype not in _INT_DTYPES:
                raise ValueError("cluster IDs must be integer tensors")
            if bool(((ids < 0) | (ids >= centers.shape[2])).any()):
                raise ValueError("external cluster IDs are out of range")
    elif previous is not None:
        kc, ki = _incremental_cluster(key, previous.key.centroids, config)
        vc, vi = _incremental_cluster(value, previous.value.centroids, config, value=True)
    else:
        kc, ki = cluster(key, config.num_clusters, config.kmeans_iterations)
        vc, vi = cluster(value, config.num_clusters, config.kmeans_iterations, value=True)
    k = _encode(key, kc, ki, plan)
    v = _encode(value, vc, vi, plan, value=True)
    if previous is not None:
        k, v = previous.key.append(k), previous.value.append(v)
    return CompressedKV(k, v)

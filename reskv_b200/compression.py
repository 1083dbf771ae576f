"""Clustering and residual compression of pre-RoPE K and V.

Public surface of the reference module (reskv/compression.py): ``cluster``,
``compress``, and the internal ``_incremental_cluster`` / ``_encode`` that
``compress`` is made of.  Every numeric step is a kernel of the native library;
this file only validates, allocates and wires results into ``CompressedTensor``.
"""

from __future__ import annotations

import torch

from ._extension import load_extension, token_stride_of
from .config import KernelPlan, ResKVKernelConfig
from .tensors import CompressedKV, CompressedTensor

_INT_DTYPES = (torch.int8, torch.int16, torch.int32, torch.int64)


def _require_kv(x, role: str) -> None:
    """K or V as the kernels read it: FP16, on a CUDA device, ``[B, H, T, 128]``, no empty axis."""
    layout_ok = isinstance(x, torch.Tensor) and x.ndim == 4 and x.shape[-1] == 128
    if not (layout_ok and x.is_cuda and x.dtype == torch.float16):
        raise ValueError(f"{role}: expected FP16 CUDA tensor [batch, kv_heads, tokens, 128]")
    if 0 in x.shape[:3]:
        raise ValueError(f"{role}: batch, head and token dimensions must be nonempty")


def _dense_or_slice(x: torch.Tensor) -> torch.Tensor:
    """``x`` itself when the kernels can address it (dense, or a token slice of a dense ``[B,H,capacity,128]``
    buffer: they take a token stride), else a dense copy."""
    return x if token_stride_of(x) is not None else x.contiguous()


def _ops(x: torch.Tensor):
    return load_extension("compression", device_index=x.device.index)


@torch.no_grad()
def cluster(x: torch.Tensor, count: int = 32, iterations: int = 10, *, value: bool = False, exact: bool = False,
            warp_mma: bool = False, return_status: bool = False):
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

    ``exact`` (not in the reference): accumulate the cluster sums as integers, which makes every mean the
    correctly rounded one.  The default (up to 32 centres) sums FP32 partials on the tensor cores in a fixed
    order -- equally reproducible, several times faster, means within one FP16 unit in the last place of the exact
    ones.  That default runs on ``tcgen05.mma`` with the token tiles brought in by TMA; ``warp_mma`` selects the
    earlier ``mma.sync`` form of the same computation, ``return_status`` appends the kernels' status word.
    """
    _require_kv(x, "cluster input")
    t = x.shape[2]
    if value:
        count = min(count, t)
    return _ops(x).kmeans(_dense_or_slice(x), int(count), int(iterations), value, exact, warp_mma, return_status)


@torch.no_grad()
def _incremental_cluster(x, centers, config, *, value=False):
    """Append the group mean as a new centre until the limit is reached, then
    assign the group's tokens (reference compression.py:56-69)."""
    append = centers.shape[2] < config.max_clusters
    return _ops(x).kmeans_incremental(_dense_or_slice(x), centers.half(), append)


@torch.no_grad()
def _encode(x, centers, ids, plan: KernelPlan, *, value=False):
    """Residuals of ``x`` to its centres in the layout of ``plan``
    (reference compression.py:72-101).  ``value`` is accepted for signature
    compatibility: K and V use the same selection rule here."""
    ids = ids.int().contiguous()
    centers = centers.half().contiguous()
    x = _dense_or_slice(x)
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


def _plan_for(config: ResKVKernelConfig, previous, plan, batch: int) -> KernelPlan:
    """The plan the new tokens are packed with: the caller's, else the existing cache's, else the
    configuration's own choice for this batch.  It has to describe the same format as ``config``."""
    if plan is None:
        plan = previous.key.plan if previous is not None else config.resolve(batch)
    asked = {"layout": config.layout, "centroid fusion": config.centroid_fusion}
    got = {"layout": plan.layout, "centroid fusion": plan.centroid_fusion}
    if (plan.bits, plan.nnz) != (config.bits, int(128 * config.keep_ratio)):
        raise ValueError("compression plan and configuration disagree")
    for what, want in asked.items():
        if want != "auto" and got[what] != want:
            raise ValueError(f"compression plan violates the requested {what}")
    if plan.fixed_shift is not (config.softmax_mode == "fixed_shift"):
        raise ValueError("compression plan and softmax configuration disagree")
    return plan


def _check_previous(previous: CompressedKV, key: torch.Tensor, limit: int) -> None:
    """An existing cache can take the new group only if it belongs to the same sequences and heads,
    lives on the same device and its centroid tables respect the configured limit."""
    tables = (previous.key.centroids, previous.value.centroids)
    same_units = previous.key.cluster_ids.shape[:2] == key.shape[:2]
    if not same_units or tables[0].device != key.device:
        raise ValueError("previous cache has incompatible dimensions or device")
    if any(t.shape[2] > limit for t in tables):
        raise ValueError("previous cache exceeds the configured centroid limit")


def _check_external(centres, ids, key: torch.Tensor, limit: int) -> None:
    """One side of ``clustering=``: a centroid table ``[B,H,C,128]`` with ``1 <= C <= limit`` and integer
    ids ``[B,H,T]`` inside ``[0, C)``, both next to K / V."""
    if centres.ndim != 4 or tuple(centres.shape[:2]) != tuple(key.shape[:2]) or centres.shape[-1] != 128:
        raise ValueError("external centers must have shape [B,H,C,128]")
    count = centres.shape[2]
    if count < 1 or count > limit or ids.shape != key.shape[:3]:
        raise ValueError("external clustering has incompatible sizes")
    if {centres.device, ids.device} != {key.device}:
        raise ValueError("external clustering must share the K/V device")
    if ids.dtype not in _INT_DTYPES:
        raise ValueError("cluster IDs must be integer tensors")
    lo, hi = torch.aminmax(ids)
    if int(lo) < 0 or int(hi) >= count:
        raise ValueError("external cluster IDs are out of range")


def _append_group_in_place(key, value, previous: CompressedKV, config, plan: KernelPlan):
    """``compress(key, value, previous=previous)`` when the new tokens can be written straight behind the live
    tokens of ``previous``'s buffers: one library call clusters the group (``_incremental_cluster``), packs it
    (``_encode``) and writes ids and packed rows in place, for K and V -- the same kernels, no intermediate
    tensors.  Returns ``None`` when ``previous`` was already extended by a sibling window (the caller then takes
    the functional path, which copies)."""
    n, t = previous.seq_len, key.shape[2]
    if previous.key._live[0] != n or previous.value._live[0] != n:
        return None
    if min(previous.key.token_stride, previous.value.token_stride) < n + t:  # full: twice the needed length
        previous = CompressedKV(*(side.reserve(max(2 * (n + t), 256)) for side in (previous.key, previous.value)))
    if token_stride_of(key) is None or token_stride_of(key) != token_stride_of(value):
        key, value = key.contiguous(), value.contiguous()
    b, h = key.shape[:2]
    sides = []
    for side in (previous.key, previous.value):
        old = side._native[0]
        count = old.shape[1]
        new = side.centroids
        if count < config.max_clusters:
            new = torch.empty((b, h, count + 1, 128), dtype=torch.float16, device=key.device)
        elif not new.is_contiguous():
            new = old.view(b, h, count, 128)
        sides.append((old, new, side._buffers))
    _ops(key).compress_group(plan, key, value, sides, n)
    windows = []
    for side, (_, new, _) in zip((previous.key, previous.value), sides):
        side._live[0] = n + t
        windows.append(side._grown(new, n + t))
    return CompressedKV(*windows)


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
    if config is None:
        config = ResKVKernelConfig()
    elif not isinstance(config, ResKVKernelConfig):
        raise TypeError("compress requires ResKVKernelConfig; ResKVConfig is for accuracy evaluation")
    _require_kv(key, "key")
    _require_kv(value, "value")
    if key.shape != value.shape or key.device != value.device:
        raise ValueError("K and V must have identical shapes and devices")
    plan = _plan_for(config, previous, plan, key.shape[0])
    if previous is not None:
        _check_previous(previous, key, config.max_clusters)
        if clustering is not None:
            raise ValueError("provide clustering or previous, not both")
    if clustering is not None:
        for centres, ids in clustering:
            _check_external(centres, ids, key, config.max_clusters)

    if previous is not None and clustering is None:
        extended = _append_group_in_place(key, value, previous, config, plan)
        if extended is not None:
            return extended

    packed = []
    for side, x in enumerate((key, value)):  # 0 = K, 1 = V
        is_value = side == 1
        if clustering is not None:
            centres, ids = clustering[side]
        elif previous is not None:
            grown = (previous.key, previous.value)[side].centroids
            centres, ids = _incremental_cluster(x, grown, config, value=is_value)
        else:
            centres, ids = cluster(x, config.num_clusters, config.kmeans_iterations, value=is_value)
        new = _encode(x, centres, ids, plan, value=is_value)
        packed.append(new if previous is None else (previous.key, previous.value)[side].append(new))
    return CompressedKV(*packed)

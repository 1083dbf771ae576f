"""Fused decode attention over a compressed cache plus the dense recent window.

``attention`` keeps the reference signature and checks
(reskv/_attention.py:10-144).  For the unstructured FP16 layout the recent
window is folded into the same two launches as the compressed tokens (partial
kernel + merge kernel) instead of the reference's extra ``bmm`` + ``mul_`` +
merge kernel.
"""

from __future__ import annotations

import torch

from ._extension import load_extension
from .config import _reference_schedule
from .tensors import CompressedKV


@torch.no_grad()
def attention(
    query: torch.Tensor,
    cache: CompressedKV,
    *,
    position: int,
    start_position: int = 0,
    rope_theta: float = 500000.0,
    inv_freq: torch.Tensor | None = None,
    scaling: float | None = None,
    recent: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
):
    """Decode raw Q against compressed pre-RoPE K and V.

    ``query`` is FP16 ``[B,H,1,128]`` before RoPE; ``recent`` is ``(rotated Q,
    rotated K, V)`` of the dense window; ``inv_freq`` holds the model's 64 RoPE
    frequencies (omit it to derive them from ``rope_theta``).  Returns FP16
    ``[B,H,1,128]``.
    """
    if query.ndim != 4 or query.shape[2:] != (1, 128) or not query.is_cuda or query.dtype != torch.float16:
        raise ValueError("query must be FP16 CUDA [batch, query_heads, 1, 128]")
    b, nh = query.shape[:2]
    kh = cache.key.centroids.shape[1]
    if query.device != cache.key.payload.device or query.device != cache.value.payload.device:
        raise ValueError("query and cache must be on the same CUDA device")
    if b != cache.key.centroids.shape[0] or cache.key.seq_len != cache.value.seq_len:
        raise ValueError("query/cache batch or K/V sequence lengths differ")
    if cache.key.plan != cache.value.plan:
        raise ValueError("K and V plans differ")
    if nh % kh or nh // kh not in (1, 4, 8):
        raise ValueError("supported query/kv head ratios are 1, 4, and 8")
    if position < start_position + cache.seq_len - 1:
        raise ValueError("query position precedes compressed tokens")
    plan = cache.key.plan
    family = "attention" if plan.centroid_fusion == "per_token" else "cluster_mass"
    ext = load_extension(family, plan, query.device.index)
    q = query.reshape(b * nh, 128).contiguous()
    kc, ki, kp, km, ks = cache.key._native
    vc, vi, vp, vm, vs = cache.value._native
    scale = 128**-0.5 if scaling is None else float(scaling)
    freq = None
    if inv_freq is not None:
        if inv_freq.shape != (64,) or inv_freq.device != query.device:
            raise ValueError("inv_freq must be [64] on the query CUDA device")
        freq = inv_freq.float().contiguous()
    has_recent = recent is not None and recent[1].shape[2] > 0
    if has_recent:
        qr, kr, vr = recent
        if qr.shape != query.shape or kr.shape != vr.shape or kr.shape[:2] != (b, kh):
            raise ValueError("recent Q/K/V shapes do not match the compressed cache")
        if any(x.device != query.device or x.dtype != torch.float16 for x in recent):
            raise ValueError("recent tensors must be FP16 on the query device")
    # A plan from ``resolve()`` carries the split count of the reference's schedule table, which was tuned
    # for other kernels on another GPU: such a plan gets this library's own schedule (0).  A split count that
    # differs from the table entry was chosen by the caller and is passed on.
    splits = plan.splits
    if plan.layout != "compact" and splits == _reference_schedule(plan.layout, plan.centroid_fusion, plan.bits, b)[1]:
        splits = 0
    suffix = (kh, nh, int(start_position), int(position), float(rope_theta), scale)
    fused = (qr.reshape(b * nh, 128), kr, vr) if has_recent else None
    # every decode op takes the dense window as an extra argument and folds it into its
    # merge kernel, so no separate merge_recent launch (or bmm) is needed here
    if plan.centroid_fusion == "deferred":
        if plan.layout == "unstructured":
            result = ext.decode_fp16(q, kc, ki, kp, km, vc, vi, vp, vm, *suffix, False, splits, freq, fused)
        else:
            fn = ext.decode_structured_int4 if plan.bits == 4 else ext.decode_structured_fp16
            result = fn(q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, *suffix, False, splits, freq, fused)
    elif plan.layout == "compact":
        result = ext.decode_compact(q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, *suffix, plan.bits, splits, freq,
                                    fused)
    elif plan.layout == "unstructured":
        result = ext.decode_quantized(q, kc, ki, kp, ks, vc, vi, vp, vs, *suffix, plan.bits, plan.bits, splits,
                                      freq, fused)
    else:
        fn = ext.decode_int4 if plan.bits == 4 else ext.decode_fp16
        result = fn(q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, *suffix, splits, freq, fused)
    return result[0].reshape(b, nh, 1, 128)

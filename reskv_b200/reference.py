"""Dense FP32 decoders and attention for checking results (not used by any kernel path).

Same three functions as the reference's verification module (reskv/reference.py:12-91), written for
this package's containers: ``reconstruct`` turns any residual layout back into dense ``[B,H,T,128]``
FP32, ``rotate`` applies half-split RoPE, ``reference_attention`` is plain softmax attention over the
reconstructed cache plus an optional dense recent window.  They run on whatever device the cache is on
with ordinary torch operators and exist so that callers (and the reference's own tests, through the
``reskv`` alias package) can verify the fused kernels; ``attention()`` never routes through them.
"""

from __future__ import annotations

import torch

from .tensors import CompressedKV, CompressedTensor


def _fields(words: torch.Tensor, bits: int, count: int) -> torch.Tensor:
    """``count`` unsigned ``bits``-wide fields per int32 word, lowest bits first -> int64 ``[..., W*count]``."""
    shifts = torch.arange(count, device=words.device) * bits
    vals = ((words.long() & 0xFFFFFFFF).unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    return vals.flatten(-2)


def _signed(codes: torch.Tensor, bits: int) -> torch.Tensor:
    sign = 1 << (bits - 1)
    return ((codes ^ sign) - sign).float()


def _expand(values: torch.Tensor, kept: torch.Tensor) -> torch.Tensor:
    """Scatter ``values[..., r]`` (ascending coordinate order) to the ``r``-th set position of ``kept``."""
    rank = (kept.long().cumsum(-1) - 1).clamp_(0, values.shape[-1] - 1)
    return torch.where(kept, values.gather(-1, rank), torch.zeros((), dtype=values.dtype, device=values.device))


def _residual(t: CompressedTensor) -> torch.Tensor:
    plan, dev = t.plan, t.payload.device
    dims = torch.arange(128, device=dev)
    if plan.layout == "compact":
        kept = ((t.metadata[..., dims // 64] >> (63 - dims % 64)) & 1).bool()
        codes = _signed(_fields(t.payload, plan.bits, 32 // plan.bits), plan.bits)
        return _expand(codes, kept) * t.scale.float().unsqueeze(-1)
    if plan.layout == "unstructured" and plan.bits != 16:
        return _signed(_fields(t.payload, plan.bits, 32 // plan.bits), plan.bits) * t.scale.float().unsqueeze(-1)
    if plan.layout == "unstructured":
        kept = ((t.metadata[..., dims // 64] >> (63 - dims % 64)) & 1).bool()
        return _expand(t.payload.float(), kept)
    if plan.bits == 4:  # one signed nibble and a 2-bit position per group of four coordinates
        codes = _signed(_fields(t.payload, 4, 8), 4) * t.scale.float().unsqueeze(-1)
        where = _fields(t.metadata, 2, 16) + torch.arange(32, device=dev) * 4
        return torch.zeros(*codes.shape[:-1], 128, device=dev).scatter_(-1, where, codes)
    tiles = _fields(t.metadata, 16, 2)  # eight 16-bit tile codes
    if plan.layout == "structured":   # four 4-bit in-tile indices per tile, payload in (tile, rank) order
        where = ((tiles.unsqueeze(-1) >> (torch.arange(4, device=dev) * 4)) & 15) + (torch.arange(8, device=dev) * 16).unsqueeze(-1)
        return torch.zeros(*t.payload.shape[:-1], 128, device=dev).scatter_(-1, where.flatten(-2), t.payload.float())
    kept = ((tiles.unsqueeze(-1) >> torch.arange(16, device=dev)) & 1).bool().flatten(-2)  # LSB-first tile masks
    return _expand(t.payload.float(), kept)


@torch.no_grad()
def reconstruct(tensor: CompressedTensor) -> torch.Tensor:
    """Dense FP32 ``[B,H,T,128]``: each token's centroid plus its decoded residual."""
    ids = tensor.cluster_ids.long().unsqueeze(-1).expand(-1, -1, -1, 128)
    return tensor.centroids.float().gather(2, ids) + _residual(tensor)


def rotate(x: torch.Tensor, positions: torch.Tensor, frequencies: torch.Tensor) -> torch.Tensor:
    """Half-split RoPE of ``x [...,P,128]`` at ``positions [P]``: coordinate ``i`` pairs with ``i + 64``."""
    angle = positions.to(x.device).float().unsqueeze(-1) * frequencies.to(x.device).float()
    cos, sin = angle.cos(), angle.sin()
    lo, hi = x.float()[..., :64], x.float()[..., 64:]
    return torch.cat((lo * cos - hi * sin, hi * cos + lo * sin), dim=-1)


@torch.no_grad()
def reference_attention(query: torch.Tensor, cache: CompressedKV, *, position: int, start_position: int = 0,
                        rope_theta: float = 500000.0, inv_freq: torch.Tensor | None = None,
                        scaling: float | None = None, recent: tuple | None = None) -> torch.Tensor:
    """FP32 attention of a pre-RoPE ``query [B,nh,1,128]`` over the reconstructed cache (keys rotated at
    ``start_position + t``, the query at ``position``) and, if given, ``recent = (rotated q, rotated k, v)``
    in one softmax -> ``[B,nh,1,128]`` float32."""
    dev = query.device
    keys, values = reconstruct(cache.key), reconstruct(cache.value)
    b, kh, t, _ = keys.shape
    nh = query.shape[1]
    freq = inv_freq.float() if inv_freq is not None else float(rope_theta) ** (-torch.arange(64, device=dev).float() / 64)
    q = rotate(query, torch.tensor([position], device=dev), freq).reshape(b, kh, nh // kh, 128)
    k = rotate(keys, torch.arange(start_position, start_position + t, device=dev), freq)
    scale = 128 ** -0.5 if scaling is None else float(scaling)
    scores = torch.matmul(q, k.transpose(-1, -2)) * scale
    if recent is not None and recent[1].shape[2] > 0:
        qr, kr, vr = recent
        scores = torch.cat((scores, torch.matmul(qr.float().reshape(b, kh, nh // kh, 128), kr.float().transpose(-1, -2)) * scale), -1)
        values = torch.cat((values, vr.float()), 2)
    return torch.matmul(torch.softmax(scores, -1), values).reshape(b, nh, 1, 128)

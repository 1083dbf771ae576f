"""Partitioning of the (sequence x KV-head) units over the GPUs of one node.

Compression and decode attention treat every (sequence, KV head) pair
independently (the reference indexes them as ``kv_idx = b * kv_heads + h``,
reskv/csrc/attention.cu:218-220), so multi-GPU execution needs no exchange on
the data path: each rank owns a contiguous range of units, the query heads of a
KV head travel with it, and outputs are concatenated in unit order.  A shard is
presented to the kernels as "one sequence with n KV heads".
"""

from __future__ import annotations

import torch


def unit_range(units: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced ``[lo, hi)`` range of ``units`` for ``rank``; the first
    ``units % world`` ranks get one unit more."""
    if units < 0 or world < 1 or not 0 <= rank < world:
        raise ValueError("need units >= 0, world >= 1 and 0 <= rank < world")
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_kv(x: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Rows of ``x [B, H, ...]`` owned by ``rank`` as ``[1, n, ...]``."""
    b, h = x.shape[:2]
    lo, hi = unit_range(b * h, world, rank)
    return x.reshape(b * h, *x.shape[2:])[lo:hi].unsqueeze(0)


def shard_query(q: torch.Tensor, kv_heads: int, world: int, rank: int) -> torch.Tensor:
    """Query heads ``[B, NH, 1, 128]`` that belong to ``rank``'s KV heads, as
    ``[1, n * (NH / KH), 1, 128]``."""
    b, nh = q.shape[:2]
    g = nh // kv_heads
    lo, hi = unit_range(b * kv_heads, world, rank)
    return q.reshape(b * kv_heads, g, *q.shape[2:])[lo:hi].reshape(1, (hi - lo) * g, *q.shape[2:])


def gather_outputs(parts: list[torch.Tensor], batch: int, q_heads: int) -> torch.Tensor:
    """Inverse of ``shard_query`` for per-rank outputs ``[1, n * g, 1, 128]`` in rank order."""
    flat = torch.cat([p.reshape(-1, *p.shape[2:]) for p in parts], dim=0)
    return flat.reshape(batch, q_heads, *flat.shape[1:])


def max_over_ranks(value: float, device=None) -> float:
    """Largest ``value`` of any rank (every rank gets it); 1-rank runs return it as is."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())

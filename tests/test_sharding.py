"""Multi-rank host logic on CPU: unit partitioning, query/output regrouping and
the max-over-ranks timing reduction, with two gloo ranks."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from reskv_b200.sharding import gather_outputs, max_over_ranks, shard_kv, shard_query, unit_range


@pytest.mark.parametrize("units,world", [(512, 8), (8, 8), (10, 4), (3, 4), (0, 2), (64, 1)])
def test_unit_ranges_partition_exactly(units, world):
    ranges = [unit_range(units, world, r) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == units
    assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    sizes = [hi - lo for lo, hi in ranges]
    assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        unit_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import attention as oatt

        b, kh, nh, t = 3, 2, 8, 40  # 6 units over 2 ranks
        g = torch.Generator().manual_seed(0)
        k = torch.randn(b, kh, t, 128, generator=g)
        v = torch.randn(b, kh, t, 128, generator=g)
        q = torch.randn(b, nh, 1, 128, generator=g).half()
        full = oatt.attention_dense(q.numpy(), k.numpy(), v.numpy(), position=t)
        ks, vs = shard_kv(k, world, rank), shard_kv(v, world, rank)
        qs = shard_query(q, kh, world, rank)
        part = torch.from_numpy(oatt.attention_dense(qs.numpy(), ks.numpy(), vs.numpy(), position=t))
        # outputs differ in size per rank in general: gather as objects
        parts = [None] * world
        dist.all_gather_object(parts, part)
        out = gather_outputs(parts, b, nh)
        slowest = max_over_ranks(10.0 + rank)
        if rank == 0:
            results.put((np.abs(out.numpy() - full).max(), slowest, [tuple(p.shape) for p in parts]))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_result():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    err, slowest, shapes = results.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err < 1e-5
    assert slowest == 11.0
    assert shapes == [(1, 12, 1, 128), (1, 12, 1, 128)]

"""A decode group appended in place (one library call for cluster + pack + write of K and V) against the
functional sequence it replaces -- ``_incremental_cluster``, ``_encode``, ``CompressedTensor.append`` -- bit
for bit, for every layout; and the window slide against slice copies."""

import pytest
import torch

from test_gpu_compress import PLANS, _plan

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _config(layout, bits, nnz, clusters, limit):
    from reskv_b200.config import ResKVKernelConfig

    return ResKVKernelConfig(sparsity=1 - nnz / 128, bits=bits, layout=layout, num_clusters=clusters, max_clusters=limit,
                             group_size=64, recent_size=32, kmeans_iterations=3)


def _functional(previous, kg, vg, config, plan):
    from reskv_b200.compression import _encode, _incremental_cluster
    from reskv_b200.tensors import CompressedKV

    packed = []
    for side, x in ((previous.key, kg), (previous.value, vg)):
        centres, ids = _incremental_cluster(x, side.centroids, config)
        packed.append(side.append(_encode(x, centres, ids, plan)))
    return CompressedKV(*packed)


def _assert_equal(a, b):
    for got, want in ((a.key, b.key), (a.value, b.value)):
        assert got.seq_len == want.seq_len
        for name in ("centroids", "cluster_ids", "payload", "metadata", "scale"):
            x, y = getattr(got, name), getattr(want, name)
            assert (x is None) == (y is None), name
            if x is not None:
                assert x.shape == y.shape and x.dtype == y.dtype, name
                assert torch.equal(x.contiguous().view(torch.uint8), y.contiguous().view(torch.uint8)), name


@pytest.mark.parametrize("layout,bits,nnz", PLANS)
def test_in_place_group_equals_the_functional_sequence(layout, bits, nnz):
    from reskv_b200 import compress
    from reskv_b200.synthetic import mixture

    config = _config(layout, bits, nnz, clusters=6, limit=8)
    plan = _plan(layout, bits, nnz)
    b, h, prompt, groups = 2, 3, 192, 4
    window = mixture(2 * b, h, prompt + 64 * groups + 40, seed=11, device=DEV)  # K then V, with room around
    k_all, v_all = window[:b], window[b:]
    fast = compress(k_all[:, :, :prompt].contiguous(), v_all[:, :, :prompt].contiguous(), config, plan=plan)
    slow = compress(k_all[:, :, :prompt].contiguous(), v_all[:, :, :prompt].contiguous(), config, plan=plan)
    fast = fast.reserve(prompt + 100)  # room for one group: the second one has to grow the buffers
    for g in range(groups):  # table grows 6 -> 7 -> 8, then stays at the limit
        lo = prompt + 64 * g
        kg, vg = k_all[:, :, lo : lo + 64], v_all[:, :, lo : lo + 64]  # token slices: strided inputs
        before = fast
        fast = compress(kg, vg, config, previous=fast, plan=plan)
        slow = _functional(slow, kg, vg, config, plan)
        torch.cuda.synchronize()
        _assert_equal(fast, slow)
        assert before.seq_len == lo and fast.seq_len == lo + 64
        assert fast.key.centroids.shape[2] == min(8, 7 + g)
    # a second continuation of an older window must not disturb the first one
    again = compress(k_all[:, :, prompt : prompt + 64], v_all[:, :, prompt : prompt + 64], config, previous=before, plan=plan)
    torch.cuda.synchronize()
    _assert_equal(fast, slow)
    assert again.seq_len == before.seq_len + 64


@pytest.mark.parametrize("cap,dst,src,count", [(96, 0, 64, 32), (96, 4, 68, 28), (160, 0, 64, 96), (40, 3, 4, 36),
                                               (96, 0, 64, 0), (17, 2, 2, 5)])
def test_window_shift_equals_slice_copies(cap, dst, src, count):
    from reskv_b200._extension import _stream, bound_library, check

    b, h = 2, 3
    bufs = torch.randn((3, b, h, cap, 128), device=DEV).half()
    want = bufs.clone()
    want[:, :, :, dst : dst + count] = bufs[:, :, :, src : src + count].clone()
    lib = bound_library(bufs.device)
    check(lib.reskv_window_shift(bufs[0].data_ptr(), bufs[1].data_ptr(), bufs[2].data_ptr(), b, h, cap, dst, src, count,
                                 _stream(bufs.device)))
    torch.cuda.synchronize()
    assert torch.equal(bufs, want)


def test_window_shift_rejects_bad_ranges():
    from reskv_b200._extension import _stream, bound_library, check

    bufs = torch.zeros((3, 1, 1, 16, 128), device=DEV).half()
    lib = bound_library(bufs.device)
    for dst, src, count in ((5, 4, 2), (0, 10, 7), (-1, 4, 2)):
        with pytest.raises(ValueError):
            check(lib.reskv_window_shift(bufs[0].data_ptr(), bufs[1].data_ptr(), bufs[2].data_ptr(), 1, 1, 16, dst, src,
                                         count, _stream(bufs.device)))

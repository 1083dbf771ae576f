"""Container behaviour that needs no GPU: appends over shared capacity buffers."""

import torch

from reskv_b200.config import KernelPlan
from reskv_b200.tensors import CompressedTensor


def _tensor(t, seed, centroids=4):
    g = torch.Generator().manual_seed(seed)
    plan = KernelPlan("unstructured", "deferred", 16, 32, 2, 0)
    return CompressedTensor(
        torch.randn(1, 2, centroids, 128, generator=g).half(),
        torch.randint(centroids, (1, 2, t), generator=g, dtype=torch.int32),
        torch.randn(1, 2, t, 32, generator=g).half(),
        torch.randint(-(2 ** 62), 2 ** 62, (1, 2, t, 2), generator=g, dtype=torch.int64),
        None, plan)


def _cat(a, b):
    return [torch.cat((x, y), 2) for x, y in ((a.cluster_ids, b.cluster_ids), (a.payload, b.payload),
                                              (a.metadata, b.metadata))]


def _same(t, want):
    return all(torch.equal(x, y) for x, y in zip((t.cluster_ids, t.payload, t.metadata), want))


def test_two_appends_from_one_parent_do_not_overwrite_each_other():
    parent, first, second, third = _tensor(100, 1), _tensor(64, 2), _tensor(64, 3), _tensor(64, 4)
    want_a, want_b = _cat(parent, first), _cat(parent, second)
    a = parent.append(first)      # grows the buffers, writes slots [100, 164)
    b = parent.append(second)     # parent's buffers are its own 100 tokens: new buffers again
    assert _same(a, want_a) and _same(b, want_b)
    # both continue in place over their own buffers ...
    a2 = a.append(third)
    assert a2.payload.data_ptr() == a.payload.data_ptr() and _same(a, want_a)
    # ... and a second continuation of `a` (whose slots behind 164 are now taken by a2) is copied
    a3 = a.append(second)
    assert a3.payload.data_ptr() != a.payload.data_ptr()
    want_a2 = [torch.cat((x, y), 2) for x, y in zip(want_a, (third.cluster_ids, third.payload, third.metadata))]
    want_a3 = [torch.cat((x, y), 2) for x, y in zip(want_a, (second.cluster_ids, second.payload, second.metadata))]
    assert _same(a2, want_a2) and _same(a3, want_a3) and _same(b, want_b)
    assert torch.equal(a3.centroids, second.centroids)  # the newer centroid table wins


def test_capacity_and_live_bytes():
    parent = _tensor(100, 5)
    grown = parent.append(_tensor(64, 6))
    per_token = 1 + 32 * 2 + 16
    assert grown.live_nbytes == 2 * 4 * 128 * 2 + 2 * 164 * per_token
    assert grown.nbytes >= grown.live_nbytes and grown.token_stride >= 2 * 164
    assert parent.live_nbytes == 2 * 4 * 128 * 2 + 2 * 100 * per_token


def test_joint_reserve_keeps_both_sides_and_shares_one_allocation():
    """CompressedKV.reserve grows K and V together: same tokens, capacity as asked, one backing storage."""
    from reskv_b200.config import KernelPlan
    from reskv_b200.tensors import CompressedKV, CompressedTensor

    plan = KernelPlan("unstructured", "deferred", 16, 32, 4, 0)
    g = torch.Generator().manual_seed(5)

    def side():
        return CompressedTensor(torch.randn(2, 3, 4, 128, generator=g).half(),
                                torch.randint(4, (2, 3, 10), generator=g, dtype=torch.int32),
                                torch.randn(2, 3, 10, 32, generator=g).half(),
                                torch.randint(1 << 40, (2, 3, 10, 2), generator=g, dtype=torch.int64), None, plan)

    kv = CompressedKV(side(), side())
    grown = kv.reserve(64)
    assert grown.seq_len == 10 and grown.key.token_stride >= 64 and grown.value.token_stride >= 64
    for a, b in ((kv.key, grown.key), (kv.value, grown.value)):
        for x, y in zip(a.tensors, b.tensors):
            assert (x is None and y is None) or torch.equal(x, y)
    storages = {t.untyped_storage().data_ptr() for t in (*grown.key._buffers, *grown.value._buffers) if t is not None}
    assert len(storages) == 1
    assert grown.reserve(32) is grown


def test_token_stride_of_recognises_token_slices_only():
    """Dense tensors and token slices of dense buffers carry a token stride; anything else does not."""
    from reskv_b200._extension import token_stride_of

    big = torch.zeros(2, 3, 50, 128, dtype=torch.float16)
    assert token_stride_of(big) == 50
    assert token_stride_of(big[:, :, 5:25]) == 50
    assert token_stride_of(big[:, :1, 5:25]) == 150          # one head per sequence: units are whole sequences apart
    assert token_stride_of(big[:1, :1, 5:25]) == 20          # a single unit: any stride will do
    assert token_stride_of(big[:, :, ::2]) is None           # every other token
    assert token_stride_of(big[:, ::2]) is None              # units no longer evenly spaced
    assert token_stride_of(big.transpose(1, 2)) is None


def test_grown_window_is_the_validated_window():
    """``_grown`` (the unchecked constructor the in-place group path uses) yields exactly the views that the
    validating ``_window`` builds over the same buffers, and shares the written-length marker."""
    base = _tensor(100, 5).reserve(400)
    newer = torch.randn(1, 2, 5, 128).half()
    fast = base._grown(newer, 164)
    slow = CompressedTensor._window(newer, base._buffers, 164, base.plan, base._live)
    assert fast.seq_len == slow.seq_len == 164 and fast.token_stride == 400 and fast._live is base._live
    for a, b in zip(fast.tensors, slow.tensors):
        assert (a is None) == (b is None)
        if a is not None:
            assert a.shape == b.shape and a.stride() == b.stride() and a.data_ptr() == b.data_ptr() and a.dtype == b.dtype
    # the old window is untouched and a further one can be derived from the new one
    assert base.seq_len == 100 and fast._grown(newer, 228).seq_len == 228

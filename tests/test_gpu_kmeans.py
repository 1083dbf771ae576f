"""CUDA Lloyd clustering against the oracle (exact nearest centre, exact means)."""

import numpy as np
import pytest
import torch

from helpers import np16
from oracle import kmeans as okm

pytestmark = pytest.mark.gpu
DEV = "cuda"
NEAR_TIE = 1e-5  # relative gap of the two smallest squared distances below which FP32 may pick either


def _cluster(x, count, iters, value=False, exact=False, warp_mma=False):
    from reskv_b200.compression import cluster

    cen, ids, status = cluster(x.to(DEV), count, iters, value=value, exact=exact, warp_mma=warp_mma, return_status=True)
    assert status == 0, f"kernel status word {status:#x}"
    return np16(cen), np16(ids)


@pytest.mark.parametrize("value", [False, True])
@pytest.mark.parametrize("count", [1, 8, 32, 64])
def test_single_iteration_is_exact(value, count):
    """One iteration: ids are the nearest initial centre (identical centroids on
    both sides, so this is the bit-exact-assignment contract); the new centres
    are the correctly rounded means."""
    from reskv_b200.synthetic import mixture

    x = mixture(2, 2, 700, seed=count, clusters=7)
    cen, ids = _cluster(x, count, 1, value, exact=True)
    want_c, want_i, margin = okm.cluster(np16(x), count, 1, value=value)
    diff = ids != want_i
    assert (margin[diff] < NEAR_TIE).all(), f"{diff.sum()} assignments differ beyond near-ties"
    if not diff.any():
        assert np.array_equal(cen.view(np.uint16), want_c.view(np.uint16))


@pytest.mark.parametrize("warp_mma", [False, True], ids=["tcgen05", "mma.sync"])
@pytest.mark.parametrize("value", [False, True])
@pytest.mark.parametrize("count,tokens", [(1, 700), (8, 700), (32, 700), (32, 3000), (20, 1025), (32, 128), (32, 5000)])
def test_tensor_core_sums_stay_within_one_fp16_ulp_of_the_exact_means(value, count, tokens, warp_mma):
    """The default accumulation (one-hot x tokens on the tensor cores, FP32 partial sums in a fixed order), in its
    tcgen05 form and in its mma.sync form: same assignments as the exact form after one iteration, every centre
    coordinate within one FP16 unit in the last place of the correctly rounded mean, and reproducible run to run."""
    from reskv_b200.synthetic import mixture

    x = mixture(2, 2, tokens, seed=count + tokens, clusters=7)
    exact_c, exact_i = _cluster(x, count, 1, value, exact=True)
    fast_c, fast_i = _cluster(x, count, 1, value, warp_mma=warp_mma)
    assert np.array_equal(fast_i, exact_i)
    a, b = fast_c.astype(np.float32), exact_c.astype(np.float32)
    assert (np.abs(a - b) <= np.spacing(np.abs(exact_c)).astype(np.float32)).all()
    assert (fast_c.view(np.uint16) != exact_c.view(np.uint16)).mean() < 0.02
    again_c, again_i = _cluster(x, count, 1, value, warp_mma=warp_mma)
    assert np.array_equal(again_c.view(np.uint16), fast_c.view(np.uint16)) and np.array_equal(again_i, fast_i)


@pytest.mark.parametrize("value", [False, True])
@pytest.mark.parametrize("shape,iterations", [((2, 4, 4133), 10), ((5, 8, 300), 10), ((8, 8, 25600), 3)],
                         ids=["ragged-tail", "many-short-units", "long-units"])
def test_both_tensor_core_forms_agree_over_a_full_run(value, shape, iterations):
    """The tcgen05 and the mma.sync form assign (almost) every token alike and end on centres within rounding of
    each other: with a ragged last tile; with units shorter than a CTA's share of tiles (a CTA of the tcgen05 form
    then crosses several unit boundaries); with units longer than the 8192 tokens one set of partial sums takes."""
    from reskv_b200.synthetic import mixture

    x = mixture(*shape, seed=17, clusters=20)
    a_c, a_i = _cluster(x, 32, iterations, value)
    b_c, b_i = _cluster(x, 32, iterations, value, warp_mma=True)
    assert (a_i != b_i).mean() < 2e-3
    np.testing.assert_allclose(a_c.astype(np.float32), b_c.astype(np.float32), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("value", [False, True])
def test_full_run_tracks_the_oracle(value):
    from reskv_b200.synthetic import mixture

    x = mixture(1, 4, 2000, seed=3, clusters=12)
    cen, ids = _cluster(x, 32, 10, value)
    want_c, want_i, margin = okm.cluster(np16(x), 32, 10, value=value)
    diff = ids != want_i
    # a near-tie early on can move a centre slightly; almost all tokens still agree
    assert diff.mean() < 2e-3
    np.testing.assert_allclose(cen.astype(np.float32), want_c.astype(np.float32), atol=5e-2, rtol=2e-2)
    assert ids.min() >= 0 and ids.max() < 32


def test_against_vectors_recorded_from_the_reference(golden):
    x = torch.from_numpy(golden["km_x"])
    for count, iters in ((8, 1), (8, 4), (32, 3)):
        cen, ids = _cluster(x, count, iters)
        ref_i, ref_c = golden[f"km_{count}_{iters}_ids"], golden[f"km_{count}_{iters}_centres"]
        assert (ids != ref_i).mean() < 5e-3
        np.testing.assert_allclose(cen.astype(np.float32), ref_c.astype(np.float32), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("count", [1, 32])
def test_value_cluster_mean_does_not_overflow(count):
    """8192 x 20.0: sums exceed FP16, means must not (reference tests/test_cuda.py:161-169)."""
    data = torch.full((1, 1, 8192, 128), 20.0, dtype=torch.float16)
    cen, ids = _cluster(data, count, 2, value=True)
    assert np.isfinite(cen.astype(np.float32)).all()
    restored = np.take_along_axis(cen, np.broadcast_to(ids.astype(np.int64)[..., None], data.shape), axis=2)
    assert np.array_equal(restored, np16(data))


def test_results_are_reproducible():
    from reskv_b200.synthetic import mixture

    x = mixture(2, 8, 3000, seed=9)
    a = _cluster(x, 32, 5)
    b = _cluster(x, 32, 5)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_incremental_step(golden):
    from reskv_b200.compression import _incremental_cluster
    from reskv_b200.config import ResKVKernelConfig

    g = golden
    cfg = ResKVKernelConfig(num_clusters=4, max_clusters=6)
    x = torch.from_numpy(g["inc_x"]).to(DEV)
    for prev_key, want_c, want_i in (("inc_prev", "inc_0_centres", "inc_0_ids"),
                                     ("inc_full_prev", "inc_full_centres", "inc_full_ids")):
        prev = torch.from_numpy(g[prev_key]).to(DEV)
        cen, ids = _incremental_cluster(x, prev, cfg)
        cen, ids = np16(cen), np16(ids)
        ref_c, ref_i = g[want_c], g[want_i]
        assert cen.shape == ref_c.shape
        n_old = g[prev_key].shape[2]
        assert np.array_equal(cen[:, :, :n_old], ref_c[:, :, :n_old])
        if cen.shape[2] > n_old:  # appended group mean: at most one FP16 ulp from torch's mean
            a, b = cen[:, :, n_old].astype(np.float32), ref_c[:, :, n_old].astype(np.float32)
            assert (np.abs(a - b) <= np.spacing(np.abs(ref_c[:, :, n_old])).astype(np.float32)).all()
        _, oi, margin = okm.incremental(g["inc_x"], g[prev_key], 6)
        assert ((ids != oi) <= (margin < 1e-3)).all()
        assert (ids != ref_i).mean() < 0.02


def test_short_inputs():
    """T < clusters: V clamps the count (reference compression.py:26); K repeats tokens."""
    from reskv_b200.synthetic import mixture

    x = mixture(1, 1, 5, seed=2)
    cen, ids = _cluster(x, 32, 3, value=True)
    assert cen.shape[2] == 5 and sorted(ids.ravel().tolist()) == [0, 1, 2, 3, 4]
    cen, ids = _cluster(x, 8, 3)
    assert cen.shape[2] == 8 and ids.max() < 8


@pytest.mark.parametrize("warp_mma", [False, True], ids=["tcgen05", "mma.sync"])
@pytest.mark.parametrize("value", [False, True])
def test_token_slice_of_a_larger_buffer_needs_no_copy(value, warp_mma):
    """x given as a token slice [:, :, 3:3+T] of a dense buffer whose other rows hold NaN: the kernels take the
    token stride, read nothing outside the slice and give the result of the dense copy."""
    from reskv_b200._extension import token_stride_of
    from reskv_b200.compression import cluster
    from reskv_b200.synthetic import mixture

    t = 1500
    dense = mixture(2, 3, t, seed=5, clusters=9).to(DEV)
    big = torch.full((2, 3, t + 40, 128), float("nan"), dtype=torch.float16, device=DEV)
    big[:, :, 3 : 3 + t] = dense
    view = big[:, :, 3 : 3 + t]
    assert not view.is_contiguous() and token_stride_of(view) == t + 40
    want_c, want_i, status = cluster(dense, 32, 3, value=value, warp_mma=warp_mma, return_status=True)
    got_c, got_i, status2 = cluster(view, 32, 3, value=value, warp_mma=warp_mma, return_status=True)
    assert status == 0 and status2 == 0
    assert torch.equal(got_i, want_i) and torch.equal(got_c.view(torch.int16), want_c.view(torch.int16))

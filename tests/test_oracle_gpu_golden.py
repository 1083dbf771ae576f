"""The CPU restatement (oracle/) against outputs recorded from the reference's own CUDA code.

``tests/golden/reference_gpu_vectors.npz`` was written by ``tests/golden/make_golden_gpu.py`` on a B200
from the reference checkout: its three CUDA packers, its device-side clustering (incl. the FP16 ``bmm``
path of V that has no CPU form) and its fused attention kernels for the eleven plans of its own test
file.  Nothing here needs a GPU."""

import numpy as np
import pytest

from oracle import attention as oatt
from oracle import encode as oenc
from oracle import kmeans as okm
from oracle import layouts as olay

from golden.make_golden_gpu import CASES, PACKER_PLANS, case_tag


@pytest.fixture(scope="module")
def g(gpu_golden):
    return gpu_golden


def _codes(words, bits):
    per = 32 // bits
    q = ((words.astype(np.int64) & 0xFFFFFFFF)[..., None] >> (np.arange(per) * bits)) & ((1 << bits) - 1)
    q = q.reshape(*words.shape[:-1], -1)
    sign = 1 << (bits - 1)
    return (q ^ sign) - sign


def _compare_packed(layout, bits, nnz, x, cen, ids, ref_payload, ref_meta, ref_scale, keep=None):
    """Oracle against recorded tensors.  Everything must be equal to the bit, except quantised codes whose
    exact quotient sits on a rounding boundary (the reference divides approximately, ``--use_fast_math``):
    those may differ by one step and are returned as ``(token index..., coordinate, oracle code, reference
    code)`` rows so that the caller can state how many there are."""
    keep = np.ones(ids.shape, bool) if keep is None else keep
    ambiguous = None
    if bits == 16:
        p, m, s = oenc.encode(layout, bits, nnz, x, cen, ids)
    elif layout == "structured":
        p, m, s, ambiguous = oenc.encode_structured_int4(x, cen, ids, return_ambiguous=True)
    else:
        (p, s, ambiguous), m = oenc.encode_quantized(x, cen, ids, nnz, bits, return_ambiguous=True), None
    if m is not None:
        assert np.array_equal(m[keep], ref_meta[keep]), "metadata differs"
    if s is not None:
        assert np.array_equal(s.view(np.uint16), ref_scale.view(np.uint16)), "scale bits differ"
    if bits == 16:
        assert np.array_equal(p[keep].view(np.uint16), ref_payload[keep].view(np.uint16)), "payload bits differ"
        return []
    mine, theirs = _codes(p, bits), _codes(ref_payload, bits)
    differ = mine != theirs
    assert not (differ & ~ambiguous).any(), "codes differ away from rounding boundaries"
    assert (np.abs(mine - theirs)[differ] == 1).all()
    return [(*idx, int(mine[tuple(idx)]), int(theirs[tuple(idx)])) for idx in np.argwhere(differ)]


@pytest.mark.parametrize("layout,bits,nnz", PACKER_PLANS)
def test_packers_bit_exact(g, layout, bits, nnz):
    """Words, metadata and scale bits of every token -- ties, zeros, extremes and subnormal rows included.
    The only codes that differ from the reference kernels' output in these 384 tokens: the exact tie
    -64 / (128 / 7) = -3.5 of the 1-of-4 INT4 packer, once per head (approximate division: -4, exact: -3)."""
    key = f"pk_{layout}_{bits}_{nnz}"
    boundary = _compare_packed(layout, bits, nnz, g["pk_x"], g["pk_cen"], g["pk_ids"], g[key + "_payload"],
                               g.get(key + "_meta"), g.get(key + "_scale"))
    expected = {("structured", 4, 32): 2}.get((layout, bits, nnz), 0)
    assert len(boundary) == expected, boundary
    if not boundary:
        p, m, s = oenc.encode(layout, bits, nnz, g["pk_x"], g["pk_cen"], g["pk_ids"])
        dense = olay.reconstruct(layout, bits, g["pk_cen"], g["pk_ids"], p, m, s)
        assert np.array_equal(dense, g[key + "_dense"])


@pytest.mark.parametrize("nnz", [32, 64])
def test_torch_encoder_on_the_device_outside_ties(g, nnz):
    p, m = oenc.encode_unstructured_fp16(g["pk_x"], g["pk_cen"], g["pk_ids"], nnz)
    keys = np.abs(oenc.residual_fp32(g["pk_x"], g["pk_cen"], g["pk_ids"]).astype(np.float16)).astype(np.float32)
    ties = oenc.tie_tokens(keys, nnz)
    assert ties.sum() < ties.size // 4
    for flavour in ("k", "v"):
        key = f"pk_unstructured_16_{nnz}_{flavour}"
        assert np.array_equal(m[~ties], g[key + "_meta"][~ties])
        assert np.array_equal(p[~ties].view(np.uint16), g[key + "_payload"][~ties].view(np.uint16))


@pytest.mark.parametrize("value", [0, 1])
@pytest.mark.parametrize("count,iters", [(8, 1), (8, 4), (32, 3), (32, 10)])
def test_device_clustering(g, value, count, iters):
    """K (FP32 cdist) and V (FP16 distances, FP16 centres) Lloyd iterations on the device.  The contract is
    the exact nearest centre; the reference's matrix-form distances (FP16 for V) may pick the other centre
    of a near-tie, which is then fed back into the means: compared are ids outside near-ties of a single
    step and, for multi-step runs, the fraction of differing ids."""
    x = g["km_x"]
    ref_c, ref_i = g[f"km_{value}_{count}_{iters}_centres"], g[f"km_{value}_{count}_{iters}_ids"]
    cen, ids, margin = okm.cluster(x, count, iters, value=bool(value))
    differ = ids != ref_i
    if iters == 1:
        tol = 2e-2 if value else 1e-4   # FP16 distance rounding of the V path is coarse
        assert not (differ & (margin > tol)).any()
        if not differ.any():
            assert np.array_equal(cen.view(np.uint16), ref_c.view(np.uint16))
    assert differ.mean() <= (0.06 if value else 0.005)
    if not differ.any():
        assert np.abs(cen.astype(np.float32) - ref_c.astype(np.float32)).max() <= 2e-3 * max(1.0, np.abs(ref_c.astype(np.float32)).max())


def test_constant_input_clusters(g):
    """8192 identical tokens (the reference's overflow case, tests/test_cuda.py:161-169)."""
    const = np.full((1, 1, 8192, 128), 20.0, np.float16)
    for count in (1, 32):
        cen, ids, _ = okm.cluster(const, count, 2, value=True)
        assert np.array_equal(ids, g[f"km_const_{count}_ids"])
        restored = np.take_along_axis(cen, np.broadcast_to(ids[..., None].astype(np.int64), const.shape), axis=2)
        assert np.array_equal(restored, const)
        ref_restored = np.take_along_axis(g[f"km_const_{count}_centres"],
                                          np.broadcast_to(g[f"km_const_{count}_ids"][..., None].astype(np.int64), const.shape), axis=2)
        assert np.array_equal(ref_restored, const)


@pytest.mark.parametrize("value", [0, 1])
def test_incremental_step_on_the_device(g, value):
    cen, ids, margin = okm.incremental(g["inc_x"], g["inc_prev"], 6, value=bool(value))
    assert np.array_equal(cen.view(np.uint16), g[f"inc_{value}_centres"].view(np.uint16))
    differ = ids != g[f"inc_{value}_ids"]
    assert not (differ & (margin > (2e-2 if value else 1e-4))).any()


def _cache(g, tag, side):
    layout, bits = tag.split("_")[1], int(tag.split("_")[2])
    return dict(layout=layout, bits=bits, centroids=g[f"at_{side}c"], ids=g[f"at_{side}i"],
                payload=g[f"{tag}_{side}_payload"], metadata=g.get(f"{tag}_{side}_meta"), scale=g.get(f"{tag}_{side}_scale"))


@pytest.mark.parametrize("bits,sparsity,layout,fusion", CASES)
def test_packed_caches_and_attention_of_the_eleven_plans(g, bits, sparsity, layout, fusion):
    """The reference's ``compress`` output for each plan is reproduced bit for bit, its FP32
    ``reference_attention`` to float rounding, and its fused kernel's output lies within the
    reference's own test tolerance of the oracle."""
    tag = "at_" + case_tag(bits, sparsity, layout, fusion)
    nnz = int(128 * (1 - sparsity))
    boundary = []
    for side, x in (("k", g["at_k"]), ("v", g["at_v"])):
        c = _cache(g, tag, side)
        keep = None
        if bits == 16 and layout == "unstructured":   # torch encoder: tie order is library-defined
            keys = np.abs(oenc.residual_fp32(x, c["centroids"], c["ids"]).astype(np.float16)).astype(np.float32)
            keep = ~oenc.tie_tokens(keys, nnz)
        boundary += _compare_packed(layout, bits, nnz, x, c["centroids"], c["ids"], c["payload"], c["metadata"],
                                    c["scale"], keep)
    # one value residual of the INT4 sparsity-0.5 cache divides to exactly 2.5 (approximate division: 3, exact: 2)
    assert len(boundary) == (1 if (bits, sparsity, layout) == (4, 0.5, "unstructured") else 0), boundary
    kc, vc = _cache(g, tag, "k"), _cache(g, tag, "v")
    for suffix, recent in (("", None), ("_recent", (g["at_qr"], g["at_kr"], g["at_vr"]))):
        want = oatt.attention_compressed(g["at_q"], kc, vc, position=288, inv_freq=g["at_freq"], recent=recent)
        np.testing.assert_allclose(want, g[tag + "_ref" + suffix], atol=2e-5, rtol=1e-4)
        np.testing.assert_allclose(g[tag + "_out" + suffix].astype(np.float32), want, atol=3e-3, rtol=3e-2)

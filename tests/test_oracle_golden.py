"""The CPU oracle against vectors recorded from the reference itself."""

import json
from pathlib import Path

import numpy as np
import pytest

from oracle import attention as oatt
from oracle import encode as oenc
from oracle import kmeans as okm
from oracle import layouts as olay

GOLD = Path(__file__).parent / "golden"

LAYOUTS = [("unstructured", 16, 32), ("unstructured", 16, 64), ("tiled", 16, 64), ("structured", 16, 32),
           ("structured", 4, 32), ("unstructured", 4, 32), ("unstructured", 4, 64), ("unstructured", 2, 32),
           ("unstructured", 2, 64)]


def _inputs(g, tag):
    return {"k": (g["x_k"], g["cen_k"], g["ids_k"]), "v": (g["x_v"], g["cen_v"], g["ids_v"]),
            "d": (g["x_distinct"], g["zero_cen"], g["zero_ids"])}[tag]


@pytest.mark.parametrize("nnz", [32, 64])
@pytest.mark.parametrize("tag", ["k", "v", "d"])
@pytest.mark.parametrize("flavour", ["k", "v"])
def test_unstructured_fp16_encoder_matches_reference(golden, nnz, tag, flavour):
    x, cen, ids = _inputs(golden, tag)
    payload, bitmap = oenc.encode_unstructured_fp16(x, cen, ids, nnz)
    ref_p = golden[f"enc_u16_{tag}_{nnz}_{flavour}_payload"]
    ref_m = golden[f"enc_u16_{tag}_{nnz}_{flavour}_meta"]
    keys = np.abs(oenc.residual_fp32(x, cen, ids).astype(np.float16)).astype(np.float32)
    ties = oenc.tie_tokens(keys, nnz)
    if tag == "d":
        assert not ties.any()
    # outside exact magnitude ties at the threshold the encodings are identical
    assert np.array_equal(bitmap[~ties], ref_m[~ties])
    assert np.array_equal(payload[~ties].view(np.uint16), ref_p[~ties].view(np.uint16))
    # inside them the reference keeps *some* coordinate of the tied magnitude:
    # the kept magnitudes agree as multisets
    a = np.sort(np.abs(payload[ties].astype(np.float32)), axis=-1)
    b = np.sort(np.abs(ref_p[ties].astype(np.float32)), axis=-1)
    assert np.array_equal(a, b)
    assert (olay.mask_unstructured_fp16(bitmap).sum(-1) == nnz).all()


@pytest.mark.parametrize("layout,bits,nnz", LAYOUTS)
def test_decoder_matches_reference_reconstruct(golden, layout, bits, nnz):
    key = f"dec_{layout}_{bits}_{nnz}"
    p = golden[key + "_payload"]
    m = golden.get(key + "_meta")
    s = golden.get(key + "_scale")
    dense = olay.reconstruct(layout, bits, golden["cen_k"], golden["ids_k"], p, m, s)
    assert np.array_equal(dense, golden[key + "_dense"])


@pytest.mark.parametrize("layout,bits,nnz", LAYOUTS)
def test_encoder_is_stable_and_obeys_the_selection_rule(golden, layout, bits, nnz):
    x, cen, ids = golden["x_k"], golden["cen_k"], golden["ids_k"]
    p, m, s = oenc.encode(layout, bits, nnz, x, cen, ids)
    key = f"dec_{layout}_{bits}_{nnz}"
    assert np.array_equal(p, golden[key + "_payload"])
    if m is not None:
        assert np.array_equal(m, golden[key + "_meta"])
    if s is not None:
        assert np.array_equal(s.view(np.uint16), golden[key + "_scale"].view(np.uint16))
    # what the reference's decoder made of those words == the rule applied directly
    r32 = oenc.residual_fp32(x, cen, ids)
    keys = np.abs(r32.astype(np.float16)).astype(np.float32)
    if layout == "unstructured":
        mask = oenc.topk_mask(keys, nnz)
    elif bits == 4:
        mask = oenc.topk_mask(keys.reshape(*keys.shape[:-1], 32, 4), 1).reshape(keys.shape)
    else:
        mask = oenc.topk_mask(keys.reshape(*keys.shape[:-1], 8, 16), nnz // 8).reshape(keys.shape)
    res = golden[key + "_dense"] - np.take_along_axis(
        cen.astype(np.float32), np.broadcast_to(ids.astype(np.int64)[..., None], r32.shape), axis=2)
    if bits == 16:
        want = np.where(mask, r32.astype(np.float16).astype(np.float32), 0)
        cenf = golden[key + "_dense"] - want
        assert np.array_equal(golden[key + "_dense"], cenf + want)
        assert np.array_equal(olay.residual(layout, bits, p, m, s), want)
    else:
        qmax = (1 << (bits - 1)) - 1
        scale = s.astype(np.float32)[..., None]
        got = olay.residual(layout, bits, p, m, s)
        assert (got[~mask] == 0).all()
        # symmetric quantiser: within half a step, never beyond qmax steps
        err = np.abs(got - r32)[mask]
        step = np.broadcast_to(scale, r32.shape)[mask]
        assert (err <= 0.5 * step * (1 + 2e-3) + 1e-6).all()
        assert (np.abs(got) <= qmax * np.broadcast_to(scale, r32.shape) * (1 + 1e-6)).all()
    del res


def test_known_answer_masks():
    """arange inputs: the reference's accuracy tests expect the top quarter of
    each token / of each 16-wide block (tests/test_accuracy.py:90-107)."""
    x = np.arange(1, 129, dtype=np.float16).reshape(1, 1, 1, 128)
    x = np.concatenate((x, -x), axis=2)
    cen = np.zeros((1, 1, 1, 128), np.float16)
    ids = np.zeros((1, 1, 2), np.int32)
    p, m = oenc.encode_unstructured_fp16(x, cen, ids, 32)
    mask = olay.mask_unstructured_fp16(m)
    assert mask[..., 96:].all() and not mask[..., :96].any()
    assert np.array_equal(p[0, 0, 0], np.arange(97, 129, dtype=np.float16))
    v, meta = oenc.encode_tiled_fp16(x, cen, ids, 32, True)
    dense = olay.residual_structured_fp16(v, meta).reshape(2, 8, 16)
    assert (np.count_nonzero(dense, axis=-1) == 4).all() and (dense[..., :12] == 0).all()
    # zero input: exact, scale 1 (compression.cu:354-355)
    z = np.zeros_like(x)
    for bits in (2, 4):
        w, s = oenc.encode_quantized(z, cen, ids, 32, bits)
        assert (w == 0).all() and (s == 1).all()
    # ties: equal magnitudes keep the lower coordinates
    ones = np.ones_like(x)
    _, m1 = oenc.encode_unstructured_fp16(ones, cen, ids, 32)
    assert olay.mask_unstructured_fp16(m1)[..., :32].all()


@pytest.mark.parametrize("nnz", [32, 64])
def test_attention_matches_reference(golden, nnz):
    g = golden
    t = g["x_k"].shape[2]

    def cache(tag, flavour):
        x, cen, ids = _inputs(g, tag)
        return dict(layout="unstructured", bits=16, centroids=cen, ids=ids,
                    payload=g[f"enc_u16_{tag}_{nnz}_{flavour}_payload"],
                    metadata=g[f"enc_u16_{tag}_{nnz}_{flavour}_meta"], scale=None)

    k, v = cache("k", "k"), cache("v", "v")
    out = oatt.attention_compressed(g["q"], k, v, position=t + 40)
    np.testing.assert_allclose(out, g[f"att_{nnz}_theta"], atol=2e-5, rtol=1e-4)
    out = oatt.attention_compressed(g["q"], k, v, position=t + 40, start_position=7,
                                    inv_freq=g["freq_model"], scaling=0.11)
    np.testing.assert_allclose(out, g[f"att_{nnz}_freq_start"], atol=2e-5, rtol=1e-4)
    rec = (g[f"att_{nnz}_qr"], g[f"att_{nnz}_kr"], g[f"att_{nnz}_vr"])
    out = oatt.attention_compressed(g["q"], k, v, position=t + 40, inv_freq=g["freq_model"], recent=rec)
    np.testing.assert_allclose(out, g[f"att_{nnz}_recent"], atol=2e-5, rtol=1e-4)


def test_rotate_matches_reference(golden):
    out = oatt.rotate(golden["q"], np.array([12345]), golden["freq_model"])
    np.testing.assert_allclose(out, golden["rotate_q"], atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("count,iters", [(8, 1), (8, 4), (32, 3)])
def test_kmeans_k_path_matches_reference(golden, count, iters):
    cen, ids, margin = okm.cluster(golden["km_x"], count, iters)
    ref_ids = golden[f"km_{count}_{iters}_ids"]
    ref_cen = golden[f"km_{count}_{iters}_centres"]
    # cdist's matrix form only disagrees with the exact nearest centre on near-ties
    diff = ids != ref_ids
    assert diff.mean() < 5e-3
    assert (margin[diff] < 1e-4).all()
    np.testing.assert_allclose(cen.astype(np.float32), ref_cen.astype(np.float32), atol=2e-2, rtol=2e-2)
    if not diff.any():
        assert np.abs(cen.astype(np.float32) - ref_cen.astype(np.float32)).max() <= 2e-3 * np.abs(ref_cen).max()


def test_kmeans_constant_input(golden):
    const = np.full((1, 1, 256, 128), 20.0, np.float16)
    cen, ids, _ = okm.cluster(const, 4, 2)
    assert np.array_equal(cen, golden["km_const_centres"])
    assert np.array_equal(ids, golden["km_const_ids"])
    cen_v, ids_v, _ = okm.cluster(const, 4, 2, value=True)
    restored = np.take_along_axis(cen_v, np.broadcast_to(ids_v.astype(np.int64)[..., None], const.shape), axis=2)
    assert np.array_equal(restored, const)


def test_incremental_matches_reference(golden):
    g = golden
    for value in (False, True):
        cen, ids, margin = okm.incremental(g["inc_x"], g["inc_prev"], 6, value=value)
        ref_c, ref_i = g[f"inc_{int(value)}_centres"], g[f"inc_{int(value)}_ids"]
        assert cen.shape == ref_c.shape == (1, 2, 6, 128)
        assert np.array_equal(cen[:, :, :5], ref_c[:, :, :5])
        assert np.abs(cen[:, :, 5].astype(np.float32) - ref_c[:, :, 5].astype(np.float32)).max() <= 2e-3
        diff = ids != ref_i
        assert (margin[diff] < (2e-2 if value else 1e-4)).all()
    cen, ids, _ = okm.incremental(g["inc_x"], g["inc_full_prev"], 6)
    assert np.array_equal(cen, g["inc_full_centres"]) and np.array_equal(ids, g["inc_full_ids"])


def test_linspace_initialisation(golden):
    off = 0
    for t, c in golden["lin_pairs"]:
        assert np.array_equal(okm.init_indices(int(t), int(c)), golden["lin_idx"][off:off + c]), (t, c)
        off += c


def test_plan_grid_matches_reference():
    from reskv_b200.config import ResKVKernelConfig

    grid = json.loads((GOLD / "plan_grid.json").read_text())
    for case in grid:
        want = case["plan"]
        try:
            got = ResKVKernelConfig(**case["settings"]).resolve(case["batch"]).to_dict()
        except ValueError as e:
            got = {"error": str(e)}
        assert got == want, case

"""CUDA residual packers against the oracle: bit-exact payloads, masks, codes
and scales given identical centroids and ids."""

import numpy as np
import pytest
import torch

from helpers import assert_packed_like_oracle, np16
from oracle import encode as oenc
from oracle import layouts as olay

pytestmark = pytest.mark.gpu
DEV = "cuda"

PLANS = [("unstructured", 16, 32), ("unstructured", 16, 64), ("tiled", 16, 64), ("structured", 16, 32),
         ("structured", 4, 32), ("unstructured", 4, 32), ("unstructured", 4, 64), ("unstructured", 2, 32),
         ("unstructured", 2, 64), ("compact", 4, 64), ("compact", 4, 32), ("compact", 2, 64)]
REFERENCE_PLANS = [p for p in PLANS if p[0] != "compact"]  # layouts the reference has (and the fixtures cover)


def _plan(layout, bits, nnz):
    from reskv_b200.config import KernelPlan

    fusion = {"unstructured": "deferred" if bits == 16 else "per_token", "tiled": "per_token",
              "structured": "deferred", "compact": "per_token"}[layout]
    return KernelPlan(layout, fusion, bits, nnz, 4, 0)


def _encode_cuda(x, cen, ids, layout, bits, nnz):
    from reskv_b200.compression import _encode

    ct = _encode(x.to(DEV), cen.to(DEV), ids.to(DEV), _plan(layout, bits, nnz))
    torch.cuda.synchronize()
    return ct


def _assert_same(ct, want):
    """Bit-exact against already packed reference tensors."""
    p, m, s = want
    got_p = np16(ct.payload)
    if got_p.dtype == np.float16:
        assert np.array_equal(got_p.view(np.uint16), p.view(np.uint16)), "payload bits differ"
    else:
        assert np.array_equal(got_p, p), "packed words differ"
    if m is None:
        assert ct.metadata is None
    else:
        assert np.array_equal(np16(ct.metadata), m), "metadata differs"
    if s is None:
        assert ct.scale is None
    else:
        assert np.array_equal(np16(ct.scale).view(np.uint16), s.view(np.uint16)), "scales differ"


def _assert_like_oracle(ct, layout, bits, nnz, x, cen, ids, boundary_limit=0.001):
    """Against the oracle on the same inputs; at most ``boundary_limit`` of the codes may sit on a rounding
    boundary of the approximate division (and then differ by one step)."""
    n = assert_packed_like_oracle(np16(ct.payload), None if ct.metadata is None else np16(ct.metadata),
                                  None if ct.scale is None else np16(ct.scale), layout, bits, nnz, np16(x), np16(cen),
                                  np16(ids))
    assert n <= boundary_limit * ids.numel() * 128, f"{n} codes on rounding boundaries"
    return n


@pytest.mark.parametrize("layout,bits,nnz", PLANS)
@pytest.mark.parametrize("shape", [(1, 1, 1, 4), (2, 3, 65, 32), (1, 2, 300, 64)])
def test_bit_exact_on_cluster_mixture(layout, bits, nnz, shape):
    from reskv_b200.synthetic import gaussian, mixture

    b, h, t, c = shape
    x = mixture(b, h, t, seed=t)
    cen = gaussian(b, h, c, 128, seed=t + 1)
    ids = torch.randint(c, (b, h, t), generator=torch.Generator().manual_seed(t + 2), dtype=torch.int32)
    ct = _encode_cuda(x, cen, ids, layout, bits, nnz)
    _assert_like_oracle(ct, layout, bits, nnz, x, cen, ids)


@pytest.mark.parametrize("layout,bits,nnz", PLANS)
def test_token_slice_of_a_larger_buffer_needs_no_copy(layout, bits, nnz):
    """x given as a token slice of a dense buffer whose other rows hold NaN: same packed bytes as the dense copy."""
    from reskv_b200._extension import token_stride_of
    from reskv_b200.compression import _encode
    from reskv_b200.synthetic import gaussian, mixture

    b, h, t, c = 2, 3, 200, 16
    x = mixture(b, h, t, seed=31).to(DEV)
    cen = gaussian(b, h, c, 128, seed=32).to(DEV)
    ids = torch.randint(c, (b, h, t), generator=torch.Generator().manual_seed(33), dtype=torch.int32).to(DEV)
    big = torch.full((b, h, t + 24, 128), float("nan"), dtype=torch.float16, device=DEV)
    big[:, :, 5 : 5 + t] = x
    view = big[:, :, 5 : 5 + t]
    assert not view.is_contiguous() and token_stride_of(view) == t + 24
    want = _encode(x, cen, ids, _plan(layout, bits, nnz))
    got = _encode(view, cen, ids, _plan(layout, bits, nnz))
    for a, w in ((got.payload, want.payload), (got.metadata, want.metadata), (got.scale, want.scale)):
        assert (a is None) == (w is None)
        if a is not None:
            assert torch.equal(a.view(torch.uint8), w.view(torch.uint8))


@pytest.mark.parametrize("layout,bits,nnz", REFERENCE_PLANS)
def test_golden_inputs_and_reference_decoder(golden, layout, bits, nnz):
    """Same inputs as the fixtures: packed output equals what the reference's
    own decoder was given, so its dense reconstruction is reproduced exactly."""
    g = golden
    x, cen, ids = (torch.from_numpy(g[k]) for k in ("x_k", "cen_k", "ids_k"))
    ct = _encode_cuda(x, cen, ids, layout, bits, nnz)
    key = f"dec_{layout}_{bits}_{nnz}"
    if _assert_like_oracle(ct, layout, bits, nnz, x, cen, ids):
        return  # a code on a rounding boundary of the approximate division: the dense tensors differ there
    _assert_same(ct, (g[key + "_payload"], g.get(key + "_meta"), g.get(key + "_scale")))
    dense = olay.reconstruct(layout, bits, g["cen_k"], g["ids_k"], np16(ct.payload),
                             None if ct.metadata is None else np16(ct.metadata),
                             None if ct.scale is None else np16(ct.scale))
    assert np.array_equal(dense, g[key + "_dense"])


@pytest.mark.parametrize("nnz", [32, 64])
def test_reference_encoder_outputs_outside_ties(golden, nnz):
    """Against the reference's own torch encoder (tie tokens excluded: their
    order is implementation-defined there)."""
    g = golden
    for tag, xs, cs, idn in (("k", "x_k", "cen_k", "ids_k"), ("v", "x_v", "cen_v", "ids_v"),
                             ("d", "x_distinct", "zero_cen", "zero_ids")):
        x, cen, ids = (torch.from_numpy(g[k]) for k in (xs, cs, idn))
        ct = _encode_cuda(x, cen, ids, "unstructured", 16, nnz)
        keys = np.abs(oenc.residual_fp32(g[xs], g[cs], g[idn]).astype(np.float16)).astype(np.float32)
        ties = oenc.tie_tokens(keys, nnz)
        for flavour in ("k", "v"):
            ref_p = g[f"enc_u16_{tag}_{nnz}_{flavour}_payload"]
            ref_m = g[f"enc_u16_{tag}_{nnz}_{flavour}_meta"]
            assert np.array_equal(np16(ct.metadata)[~ties], ref_m[~ties])
            assert np.array_equal(np16(ct.payload)[~ties].view(np.uint16), ref_p[~ties].view(np.uint16))


@pytest.mark.parametrize("layout,bits,nnz", PLANS)
def test_ties_zeros_and_extremes(layout, bits, nnz):
    rows = [np.ones(128), np.zeros(128), -np.ones(128) * 3, np.arange(1, 129), -np.arange(1, 129)[::-1],
            np.tile([5, 5, -5, 5, 1, 1, 1, 1], 16), np.full(128, 60000.0), np.full(128, 6e-8),
            np.tile([6e-8, 0, -6e-8, 1.2e-7], 32)]
    x = torch.tensor(np.stack(rows), dtype=torch.float16).reshape(1, 1, len(rows), 128)
    cen = torch.zeros(1, 1, 2, 128, dtype=torch.float16)
    cen[0, 0, 1] = 0.5
    ids = torch.tensor([i % 2 for i in range(len(rows))], dtype=torch.int32).reshape(1, 1, -1)
    # the last row (zero centre, subnormal residuals) makes the INT4 scale fp16(1.2e-7 / 7) underflow to 0: the
    # quotients are +-inf / NaN and the codes the low half of the saturated 64-bit conversion -- -1 for positive
    # residuals, 0 otherwise -- which is what the reference's `(int)lrintf(r / 0)` stores
    ct = _encode_cuda(x, cen, ids, layout, bits, nnz)
    _assert_like_oracle(ct, layout, bits, nnz, x, cen, ids, boundary_limit=0.01)
    if bits == 4 and layout == "unstructured":
        from helpers import unpack_codes

        assert np16(ct.scale)[0, 0, -1] == 0
        codes = unpack_codes(np16(ct.payload), 4)[0, 0, -1]
        assert set(codes.tolist()) == {-1, 0} and (codes[3::4] == -1).all() and (codes[2::4] == 0).all()


@pytest.mark.parametrize("bits,nnz", [(4, 64), (4, 32), (2, 64)])
def test_compact_layout_holds_the_codes_of_the_quantised_layout(bits, nnz):
    """The compact layout stores the same codes as the unstructured quantised layout, kept
    coordinates only: both decode to the same dense residual, in 16 + nnz*bits/8 bytes per token."""
    from reskv_b200.synthetic import gaussian, mixture

    x = mixture(2, 2, 200, seed=5)
    cen = gaussian(2, 2, 16, 128, seed=6)
    ids = torch.randint(16, (2, 2, 200), generator=torch.Generator().manual_seed(7), dtype=torch.int32)
    compact = _encode_cuda(x, cen, ids, "compact", bits, nnz)
    full = _encode_cuda(x, cen, ids, "unstructured", bits, nnz)
    a = olay.residual("compact", bits, np16(compact.payload), np16(compact.metadata), np16(compact.scale))
    b = olay.residual("unstructured", bits, np16(full.payload), None, np16(full.scale))
    assert np.array_equal(a, b)
    assert compact.payload.shape[-1] * 4 == nnz * bits // 8 and compact.metadata.shape[-1] == 2


def test_out_of_range_ids_are_rejected():
    from reskv_b200 import compress
    from reskv_b200.synthetic import gaussian

    k = gaussian(1, 1, 64, 128, seed=1, device=DEV)
    cen = gaussian(1, 1, 32, 128, seed=2, device=DEV)
    ids = torch.randint(32, (1, 1, 64), device=DEV, dtype=torch.int32)
    ids[0, 0, 0] = 32
    with pytest.raises(ValueError, match="out of range"):
        compress(k, k, clustering=((cen, ids), (cen, ids)))
    with pytest.raises(TypeError, match="compress requires ResKVKernelConfig"):
        compress(k, k, {})


def test_full_size_properties():
    """BASELINE-sized head (8128 tokens): properties that need no oracle run.
    Kept count, kept >= dropped magnitudes, payload == fp16 residual, and the
    quantised codes stay within half a step."""
    from reskv_b200.compression import _encode
    from reskv_b200.synthetic import gaussian, mixture

    b, h, t, c = 2, 8, 8128, 32
    x = mixture(b, h, t, seed=5, device=DEV)
    cen = gaussian(b, h, c, 128, seed=6, device=DEV)
    ids = torch.randint(c, (b, h, t), device=DEV, dtype=torch.int32)
    r = x.float() - torch.gather(cen.float(), 2, ids.long().unsqueeze(-1).expand(-1, -1, -1, 128))
    key = r.half().abs().float()
    for nnz in (32, 64):
        ct = _encode(x, cen, ids, _plan("unstructured", 16, nnz))
        dims = torch.arange(128, device=DEV)
        mask = ((ct.metadata[..., dims // 64] >> (63 - dims % 64)) & 1).bool()
        assert (mask.sum(-1) == nnz).all()
        kept_min = torch.where(mask, key, torch.full_like(key, float("inf"))).amin(-1)
        drop_max = torch.where(mask, torch.zeros_like(key), key).amax(-1)
        assert (kept_min >= drop_max).all()
        rank = mask.long().cumsum(-1) - 1
        dense = torch.where(mask, ct.payload.gather(-1, rank.clamp_min(0)), torch.zeros_like(x))
        assert torch.equal(dense, torch.where(mask, r.half(), torch.zeros_like(x)))
        q = _encode(x, cen, ids, _plan("unstructured", 4, nnz))
        shifts = torch.arange(8, device=DEV) * 4
        codes = ((q.payload.long().unsqueeze(-1) >> shifts) & 15).reshape(b, h, t, 128)
        codes = (codes ^ 8) - 8
        assert torch.equal(codes != 0, (codes != 0) & mask)
        err = (codes.float() * q.scale.float().unsqueeze(-1) - r).abs()
        step = q.scale.float().unsqueeze(-1).expand_as(r)
        assert (err[mask] <= 0.5 * step[mask] * 1.002 + 1e-6).all()

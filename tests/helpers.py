"""Glue between torch tensors of the package and the numpy oracle."""

import numpy as np
import torch

from oracle import attention as oatt
from oracle import encode as oenc

ATOL, RTOL = 2e-3, 1e-2  # attention outputs: |a - b| <= ATOL + RTOL * |b|


def np16(t):
    return t.detach().cpu().numpy()


def oracle_cache(x, cen, ids, layout, bits, nnz):
    """Encode with the oracle -> dict the oracle's attention understands."""
    p, m, s = oenc.encode(layout, bits, nnz, np16(x), np16(cen), np16(ids))
    return dict(layout=layout, bits=bits, centroids=np16(cen), ids=np16(ids), payload=p, metadata=m, scale=s)


def to_compressed(cache: dict, plan, device):
    """Oracle-encoded dict -> CompressedTensor on ``device``."""
    from reskv_b200.tensors import CompressedTensor

    def dev(a):
        return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(device)

    return CompressedTensor(dev(cache["centroids"]), dev(cache["ids"]), dev(cache["payload"]), dev(cache["metadata"]),
                            dev(cache["scale"]), plan)


def oracle_attention(q, kcache, vcache, **kw):
    recent = kw.pop("recent", None)
    if recent is not None:
        recent = tuple(np16(r) for r in recent)
    inv_freq = kw.pop("inv_freq", None)
    if inv_freq is not None:
        inv_freq = np16(inv_freq)
    return oatt.attention_compressed(np16(q), kcache, vcache, recent=recent, inv_freq=inv_freq, **kw)


def assert_attention_close(got, want, atol=ATOL, rtol=RTOL):
    got = got.detach().float().cpu().numpy().reshape(want.shape)
    err = np.abs(got - want)
    bound = atol + rtol * np.abs(want)
    worst = (err - bound).max()
    assert worst <= 0, f"max abs err {err.max():.3e}, worst excess over tolerance {worst:.3e}"


def unpack_codes(words, bits):
    """Signed ``bits``-wide fields of int32 words, lowest bits first -> int64 ``[..., W * 32 / bits]``."""
    per = 32 // bits
    q = ((words.astype(np.int64) & 0xFFFFFFFF)[..., None] >> (np.arange(per) * bits)) & ((1 << bits) - 1)
    q = q.reshape(*words.shape[:-1], -1)
    sign = 1 << (bits - 1)
    return (q ^ sign) - sign


def assert_packed_like_oracle(payload, metadata, scale, layout, bits, nnz, x, cen, ids):
    """CUDA packer output (numpy arrays) against the oracle: payload / metadata / scale equal to the bit.

    Quantised codes are compared as integers; a code may differ by one step only where the exact quotient
    sits on a rounding boundary (the kernels divide approximately like the reference's fast-math build, the
    oracle divides exactly; ``oracle.encode.near_half_integer``).  Returns the number of such codes."""
    if bits == 16:
        p, m, s = oenc.encode(layout, bits, nnz, x, cen, ids)
        assert np.array_equal(payload.view(np.uint16), p.view(np.uint16)), "payload bits differ"
        assert np.array_equal(metadata, m), "metadata differs"
        assert scale is None
        return 0
    if layout == "structured":
        p, m, s, ambiguous = oenc.encode_structured_int4(x, cen, ids, return_ambiguous=True)
        mine, want = unpack_codes(payload, 4), unpack_codes(p, 4)
    else:
        p, s, ambiguous = oenc.encode_quantized(x, cen, ids, nnz, bits, return_ambiguous=True)
        m = None
        if layout == "compact":
            _, m, _ = oenc.encode_compact(x, cen, ids, nnz, bits)
            # codes of the kept coordinates only: expand both to all 128 coordinates by the (identical) bitmap
            assert np.array_equal(metadata, m), "bitmap differs"
            from oracle import layouts as olay

            one = np.ones(scale.shape, np.float16)
            mine = olay.residual_compact(payload, metadata, one, bits).astype(np.int64)
            want = unpack_codes(p, bits)
        else:
            mine, want = unpack_codes(payload, bits), unpack_codes(p, bits)
    if m is None:
        assert metadata is None
    elif layout != "compact":
        assert np.array_equal(metadata, m), "metadata differs"
    assert np.array_equal(scale.view(np.uint16), s.view(np.uint16)), "scale bits differ"
    differ = mine != want
    assert not (differ & ~ambiguous).any(), "codes differ away from rounding boundaries"
    assert (np.abs(mine - want)[differ] == 1).all()
    return int(differ.sum())

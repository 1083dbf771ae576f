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

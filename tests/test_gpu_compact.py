"""Decode attention over the compact quantised layout (bitmap + codes of the retained
coordinates; not in the reference) against the FP32 oracle, through the public API."""

import numpy as np
import pytest
import torch

from helpers import assert_attention_close, np16, oracle_attention
from oracle import attention as oatt

pytestmark = pytest.mark.gpu
DEV = "cuda"
PLANS = [(4, 0.5), (4, 0.75), (2, 0.5)]


def _as_oracle(ct):
    p = ct.plan
    return dict(layout=p.layout, bits=p.bits, centroids=np16(ct.centroids), ids=np16(ct.cluster_ids),
                payload=np16(ct.payload), metadata=np16(ct.metadata), scale=np16(ct.scale))


def _reference(q, cache, **kw):
    return oracle_attention(q, _as_oracle(cache.key), _as_oracle(cache.value), **kw)


@pytest.mark.parametrize("bits,sparsity", PLANS)
@pytest.mark.parametrize("t,gqa", [(1, 4), (65, 1), (1000, 4), (2500, 8)])
def test_attention_matches_the_oracle(bits, sparsity, t, gqa):
    from reskv_b200 import ResKVKernelConfig, attention, compress
    from reskv_b200.synthetic import gaussian, mixture

    b, h = 2, 2
    k, v = mixture(b, h, t, seed=t), mixture(b, h, t, seed=t + 1)
    q = gaussian(b, h * gqa, 1, 128, seed=t + 2)
    cen = gaussian(b, h, 32, 128, seed=t + 3)
    ids = torch.randint(32, (b, h, t), generator=torch.Generator().manual_seed(t), dtype=torch.int32)
    cfg = ResKVKernelConfig(bits=bits, sparsity=sparsity, layout="compact")
    clustering = tuple((cen.to(DEV), ids.to(DEV)) for _ in range(2))
    cache = compress(k.to(DEV), v.to(DEV), cfg, clustering=clustering)
    assert cache.key.plan.layout == "compact"
    out = attention(q.to(DEV), cache, position=t + 10, start_position=3)
    assert_attention_close(out, _reference(q, cache, position=t + 10, start_position=3))


@pytest.mark.parametrize("bits,sparsity", PLANS)
def test_recent_window_model_frequencies_and_clustered_pipeline(bits, sparsity):
    from reskv_b200 import ResKVKernelConfig, attention, compress
    from reskv_b200.synthetic import gaussian, mixture

    b, h, t, live = 1, 3, 704, 40
    k, v = mixture(b, h, t + live, seed=11), mixture(b, h, t + live, seed=12)
    q = gaussian(b, h * 4, 1, 128, seed=13)
    cfg = ResKVKernelConfig(bits=bits, sparsity=sparsity, layout="compact", kmeans_iterations=4)
    cache = compress(k[:, :, :t].contiguous().to(DEV), v[:, :, :t].contiguous().to(DEV), cfg)
    freq = (1e6 ** (-torch.arange(64).float() / 64)).float()
    pos = t + live - 1
    qr = torch.from_numpy(oatt.rotate(np16(q), np.array([pos]), np16(freq))).half()
    kr = torch.from_numpy(oatt.rotate(np16(k[:, :, t:]), np.arange(t, t + live), np16(freq))).half()
    vr = v[:, :, t:].contiguous()
    kw = dict(position=pos, inv_freq=freq, scaling=0.1)
    out = attention(q.to(DEV), cache, recent=tuple(x.to(DEV) for x in (qr, kr, vr)), **{**kw, "inv_freq": freq.to(DEV)})
    assert_attention_close(out, _reference(q, cache, recent=(qr, kr, vr), **kw))


def test_compact_cache_is_smaller_and_appends_in_place():
    from reskv_b200 import ResKVKernelConfig, compress
    from reskv_b200.synthetic import mixture

    k, v = mixture(1, 2, 256, seed=1).to(DEV), mixture(1, 2, 256, seed=2).to(DEV)
    sizes = {}
    for layout in ("compact", "unstructured"):
        cfg = ResKVKernelConfig(bits=4, sparsity=0.5, layout=layout, kmeans_iterations=2)
        cache = compress(k[:, :, :192].contiguous(), v[:, :, :192].contiguous(), cfg)
        grown = compress(k[:, :, 192:].contiguous(), v[:, :, 192:].contiguous(), cfg, previous=cache)
        assert grown.seq_len == 256
        sizes[layout] = cache.key.payload.shape[-1] * 4 + (16 if layout == "compact" else 0) + 2 + 1
    assert sizes == {"compact": 51, "unstructured": 67}


def test_no_warp_per_token_kernel():
    from reskv_b200 import ResKVKernelConfig, attention, compress
    from reskv_b200._extension import library
    from reskv_b200.synthetic import gaussian, mixture

    k, v = mixture(1, 1, 64, seed=1).to(DEV), mixture(1, 1, 64, seed=2).to(DEV)
    cache = compress(k, v, ResKVKernelConfig(bits=4, sparsity=0.5, layout="compact", kmeans_iterations=1))
    lib = library()
    lib.reskv_decode_set_variant(1)
    try:
        with pytest.raises(ValueError, match="no warp-per-token kernel"):
            attention(gaussian(1, 4, 1, 128, seed=3, device=DEV), cache, position=64)
    finally:
        lib.reskv_decode_set_variant(0)

"""The public API end to end on the GPU, structured like the reference's own
CUDA tests (tests/test_cuda.py): compress -> attention against the FP32 oracle
for every (bits, sparsity, layout, fusion) plan, streams, incremental cache,
GQA ratios, argument errors."""

import numpy as np
import pytest
import torch

from helpers import assert_attention_close, np16, oracle_attention
from oracle import attention as oatt
from oracle import layouts as olay

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True, params=["tensor-core", "simt"])
def kernel_variant(request):
    """Every test runs with both families of partial kernels."""
    from reskv_b200._extension import library

    lib = library()
    assert lib.reskv_decode_set_variant(0 if request.param == "tensor-core" else 1) == 0
    yield request.param
    lib.reskv_decode_set_variant(0)

CASES = [
    (16, 0.5, "tiled", "per_token"),
    (16, 0.5, "unstructured", "deferred"),
    (16, 0.75, "unstructured", "deferred"),
    (16, 0.75, "structured", "per_token"),
    (16, 0.75, "structured", "deferred"),
    (4, 0.5, "unstructured", "per_token"),
    (4, 0.75, "unstructured", "per_token"),
    (4, 0.75, "structured", "per_token"),
    (4, 0.75, "structured", "deferred"),
    (2, 0.5, "unstructured", "per_token"),
    (2, 0.75, "unstructured", "per_token"),
]


def inputs(b=1, t=256, heads=1, gqa=4, clusters=32, seed=123):
    g = torch.Generator().manual_seed(seed)
    k = (torch.randn(b, heads, t, 128, generator=g) * 0.5).half()
    v = (torch.randn(b, heads, t, 128, generator=g) * 0.5).half()
    q = (torch.randn(b, heads * gqa, 1, 128, generator=g) * 0.5).half()
    kc = (torch.randn(b, heads, clusters, 128, generator=g) * 0.1).half()
    vc = (torch.randn(b, heads, clusters, 128, generator=g) * 0.1).half()
    ki = torch.randint(clusters, (b, heads, t), generator=g, dtype=torch.int32)
    vi = torch.randint(clusters, (b, heads, t), generator=g, dtype=torch.int32)
    return k, v, q, ((kc, ki), (vc, vi))


def cuda(x):
    if isinstance(x, tuple):
        return tuple(cuda(y) for y in x)
    return x.to(DEV)


def as_oracle(ct):
    p = ct.plan
    return dict(layout=p.layout, bits=p.bits, centroids=np16(ct.centroids), ids=np16(ct.cluster_ids),
                payload=np16(ct.payload), metadata=None if ct.metadata is None else np16(ct.metadata),
                scale=None if ct.scale is None else np16(ct.scale))


def reference(q, cache, **kw):
    return oracle_attention(q, as_oracle(cache.key), as_oracle(cache.value), **kw)


@pytest.mark.parametrize("bits,sparsity,layout,fusion", CASES)
def test_fused_and_mixed_against_fp32(bits, sparsity, layout, fusion):
    from reskv_b200 import ResKVKernelConfig, attention, compress

    k, v, q, clustering = inputs()
    cfg = ResKVKernelConfig(bits=bits, sparsity=sparsity, layout=layout, centroid_fusion=fusion)
    cache = compress(cuda(k), cuda(v), cfg, clustering=cuda(clustering))
    # non-standard frequencies catch kernels that hard-code the RoPE theta
    freq = (500000.0 ** (-torch.arange(64).float() / 64) / torch.linspace(1, 8, 64)).float()
    out = attention(cuda(q), cache, position=288, inv_freq=cuda(freq))
    assert_attention_close(out, reference(q, cache, position=288, inv_freq=freq))
    g = torch.Generator().manual_seed(7)
    kr = (torch.randn(1, 1, 32, 128, generator=g) * 0.5).half()
    vr = (torch.randn(1, 1, 32, 128, generator=g) * 0.5).half()
    qr = torch.from_numpy(oatt.rotate(np16(q), np.array([288]), np16(freq))).half()
    mixed = attention(cuda(q), cache, position=288, inv_freq=cuda(freq), recent=cuda((qr, kr, vr)))
    assert_attention_close(mixed, reference(q, cache, position=288, inv_freq=freq, recent=(qr, kr, vr)))


@pytest.mark.parametrize("bits,sparsity,layout,fusion", CASES)
@pytest.mark.parametrize("t", [1, 65, 1000])
def test_every_plan_on_outlier_channels_and_odd_lengths(bits, sparsity, layout, fusion, t):
    """Cluster-mixture inputs with log-normal channel scales, lengths that are
    not multiples of the tile, two sequences x three KV heads, theta RoPE."""
    from reskv_b200 import ResKVKernelConfig, attention, compress
    from reskv_b200.synthetic import gaussian, mixture

    b, h = 2, 3
    k, v = mixture(b, h, t, seed=t), mixture(b, h, t, seed=t + 1)
    q = gaussian(b, h * 4, 1, 128, seed=t + 2)
    cen = gaussian(b, h, 32, 128, seed=t + 3)
    ids = torch.randint(32, (b, h, t), generator=torch.Generator().manual_seed(t), dtype=torch.int32)
    cfg = ResKVKernelConfig(bits=bits, sparsity=sparsity, layout=layout, centroid_fusion=fusion)
    cache = compress(cuda(k), cuda(v), cfg, clustering=cuda(((cen, ids), (cen, ids))))
    out = attention(cuda(q), cache, position=t + 10, start_position=3)
    assert_attention_close(out, reference(q, cache, position=t + 10, start_position=3))


@pytest.mark.parametrize("bits,layout", [(16, "unstructured"), (16, "structured"), (4, "unstructured"),
                                         (4, "structured"), (2, "unstructured")])
def test_current_stream(bits, layout):
    from reskv_b200 import ResKVKernelConfig, attention, compress

    stream = torch.cuda.Stream()
    k, v, q, c = inputs(t=64)
    with torch.cuda.stream(stream):
        cache = compress(cuda(k), cuda(v), ResKVKernelConfig(bits=bits, sparsity=0.75, layout=layout),
                         clustering=cuda(c))
        out = attention(cuda(q), cache, position=64)
    stream.synchronize()
    assert_attention_close(out, reference(q, cache, position=64), atol=3e-3)


def test_incremental_cache_no_tokens_lost_and_centroids_capped():
    from reskv_b200 import ResKVKernelConfig
    from reskv_b200.cache import ResKVLayerCache

    cfg = ResKVKernelConfig(bits=16, layout="unstructured", num_clusters=4, max_clusters=6, group_size=16,
                            recent_size=8)
    cache = ResKVLayerCache(cfg)
    k, v, _, _ = inputs(t=35)
    k, v = cuda(k), cuda(v)
    cache.update(k, v, {"raw_keys": k})
    assert cache.compressed.seq_len + cache.live == 35
    for _ in range(100):
        token = k[:, :, :1]
        cache.update(token, token, {"raw_keys": token})
        assert cache.compressed.seq_len + cache.live == cache.length
        assert cache.compressed.key.centroids.shape[2] <= 6
    assert cache.length == 135
    cache.reset()
    assert cache.get_seq_length() == 0 and cache.compressed is None


def test_incremental_cache_matches_one_shot_attention():
    """Decode 200 tokens through the cache (prefill + 3 group compressions) and
    compare attention over (compressed + window) with the oracle on the same
    compressed tensors."""
    from reskv_b200 import ResKVKernelConfig, attention
    from reskv_b200.cache import ResKVLayerCache
    from reskv_b200.synthetic import gaussian, mixture

    cfg = ResKVKernelConfig(sparsity=0.75, layout="unstructured", kmeans_iterations=3)
    b, h, t0 = 2, 2, 300
    k, v = mixture(b, h, t0 + 200, seed=5), mixture(b, h, t0 + 200, seed=6)
    freq = oatt.theta_frequencies(500000.0)

    def rot(x, start):
        return torch.from_numpy(oatt.rotate(np16(x), np.arange(start, start + x.shape[2]), freq)).half()

    layer = ResKVLayerCache(cfg)
    layer.update(cuda(rot(k[:, :, :t0], 0)), cuda(v[:, :, :t0]), {"raw_keys": cuda(k[:, :, :t0])})
    for i in range(t0, t0 + 200):
        keys, values = layer.update(cuda(rot(k[:, :, i:i + 1], i)), cuda(v[:, :, i:i + 1]),
                                    {"raw_keys": cuda(k[:, :, i:i + 1])})
    assert layer.compressed.seq_len + layer.live == t0 + 200
    assert layer.compressed.seq_len == (t0 - 32) // 64 * 64 + 3 * 64
    assert layer.compressed.key.centroids.shape[2] == 35
    pos = t0 + 199
    q = gaussian(b, h * 4, 1, 128, seed=9)
    qr = torch.from_numpy(oatt.rotate(np16(q), np.array([pos]), freq)).half()
    out = attention(cuda(q), layer.compressed, position=pos, recent=(cuda(qr), keys, values))
    want = reference(q, layer.compressed, position=pos, recent=(qr, keys.cpu(), values.cpu()))
    assert_attention_close(out, want)
    # the dense window holds exactly the most recent tokens
    n = layer.compressed.seq_len
    assert torch.equal(values.cpu(), v[:, :, n:])


def test_cache_with_sink_tokens_at_the_reference_cpu_configuration():
    """One Llama-3.1-8B-shaped layer, batch 1, 8 KV heads, context 8192, 4 sink tokens, window 32, group 64,
    sparsity 0.5: the prompt splits into 4 sinks + 8128 compressed tokens + 60 dense ones; 70 more tokens cross
    one group compression.  Attention over (sinks + compressed + window) equals dense attention over the
    reconstructed cache at the original positions."""
    from reskv_b200 import ResKVKernelConfig, attention
    from reskv_b200.cache import ResKVLayerCache
    from reskv_b200.synthetic import gaussian, mixture

    cfg = ResKVKernelConfig(sparsity=0.5, layout="unstructured", kmeans_iterations=10, num_clusters=32)
    b, h, t0, extra, sinks = 1, 8, 8192, 70, 4
    k, v = mixture(b, h, t0 + extra, seed=21), mixture(b, h, t0 + extra, seed=22)
    freq = oatt.theta_frequencies(500000.0)

    def rot(x, start):
        return torch.from_numpy(oatt.rotate(np16(x), np.arange(start, start + x.shape[2]), freq)).half()

    layer = ResKVLayerCache(cfg, sink_tokens=sinks)
    keys, values = layer.update(cuda(rot(k[:, :, :t0], 0)), cuda(v[:, :, :t0]), {"raw_keys": cuda(k[:, :, :t0])})
    assert layer.start_position == sinks and layer.compressed.seq_len == 8128 and layer.live == sinks + 60
    assert torch.equal(values[:, :, :sinks].cpu(), v[:, :, :sinks]) and torch.equal(values[:, :, sinks:].cpu(), v[:, :, sinks + 8128:t0])
    for i in range(t0, t0 + extra):
        keys, values = layer.update(cuda(rot(k[:, :, i:i + 1], i)), cuda(v[:, :, i:i + 1]),
                                    {"raw_keys": cuda(k[:, :, i:i + 1])})
    n = layer.compressed.seq_len
    assert n == 8128 + 64 and layer.live == sinks + (t0 + extra - sinks - n)
    assert torch.equal(values.cpu(), torch.cat((v[:, :, :sinks], v[:, :, sinks + n:]), 2))
    assert torch.equal(keys[:, :, :sinks].cpu(), rot(k[:, :, :sinks], 0))
    pos = t0 + extra - 1
    q = gaussian(b, h * 4, 1, 128, seed=23)
    qr = torch.from_numpy(oatt.rotate(np16(q), np.array([pos]), freq)).half()
    out = attention(cuda(q), layer.compressed, position=pos, start_position=layer.start_position,
                    recent=(cuda(qr), keys, values))
    want = reference(q, layer.compressed, position=pos, start_position=sinks, recent=(qr, keys.cpu(), values.cpu()))
    assert_attention_close(out, want)
    with pytest.raises(ValueError, match="sink_tokens"):
        ResKVLayerCache(cfg, sink_tokens=-1)


def test_layouts_have_different_selection_semantics():
    from reskv_b200 import ResKVKernelConfig, compress

    k, v, _, c = inputs(t=64)
    u = compress(cuda(k), cuda(v), ResKVKernelConfig(bits=16, sparsity=0.75, layout="unstructured"), clustering=cuda(c))
    s = compress(cuda(k), cuda(v), ResKVKernelConfig(bits=16, sparsity=0.75, layout="structured"), clustering=cuda(c))
    assert not np.array_equal(olay.reconstruct(**as_oracle(u.key)), olay.reconstruct(**as_oracle(s.key)))
    assert u.key.payload.shape[-1] == s.key.payload.shape[-1] == 32


@pytest.mark.parametrize("ratio", [1, 8])
@pytest.mark.parametrize("bits,layout", [(16, "unstructured"), (16, "structured"), (4, "structured"),
                                         (2, "unstructured")])
def test_gqa_and_64_centroids(ratio, bits, layout):
    from reskv_b200 import ResKVKernelConfig, attention, compress

    k, v, q, _ = inputs(t=320)
    q = q[:, :1].repeat(1, ratio, 1, 1)
    centers = k[:, :, :64].contiguous()
    ids = torch.arange(320, dtype=torch.int32).remainder(64).view(1, 1, -1)
    cfg = ResKVKernelConfig(bits=bits, sparsity=0.75, layout=layout)
    cache = compress(cuda(k), cuda(v), cfg, clustering=cuda(((centers, ids), (centers, ids))))
    out = attention(cuda(q), cache, position=330, start_position=10)
    assert_attention_close(out, reference(q, cache, position=330, start_position=10))


def test_structured_int4_stable_softmax_large_logits():
    from reskv_b200 import ResKVKernelConfig, attention, compress

    k, v, q, c = inputs(t=256)
    k, q = k * 12, q * 12
    cfg = ResKVKernelConfig(bits=4, sparsity=0.75, layout="structured", centroid_fusion="deferred")
    cache = compress(cuda(k), cuda(v), cfg, clustering=cuda(c))
    out = attention(cuda(q), cache, position=256)
    assert out.isfinite().all()
    assert_attention_close(out, reference(q, cache, position=256), atol=2e-2, rtol=5e-2)


def test_theta_rope_with_model_rotated_recent_tokens():
    from reskv_b200 import ResKVKernelConfig, attention, compress

    k, v, q, c = inputs(t=256)
    cfg = ResKVKernelConfig(bits=4, sparsity=0.75, layout="unstructured", rope_mode="theta")
    cache = compress(cuda(k), cuda(v), cfg, clustering=cuda(c))
    model_freq = (500000.0 ** (-torch.arange(64).float() / 64) / 8).float()
    qr = torch.from_numpy(oatt.rotate(np16(q), np.array([288]), np16(model_freq))).half()
    recent = (qr, k[:, :, :32].contiguous(), v[:, :, :32].contiguous())
    out = attention(cuda(q), cache, position=288, recent=cuda(recent))
    assert_attention_close(out, reference(q, cache, position=288, recent=recent))


def test_full_clustered_pipeline_against_dense_attention():
    """compress() with its own K-means, sparsity 0.5: the compressed attention
    stays close to dense attention on the same K/V (informational bound, the
    gate is the oracle comparison on the compressed tensors)."""
    from reskv_b200 import ResKVKernelConfig, attention, compress
    from reskv_b200.synthetic import gaussian, mixture

    b, h, t = 1, 8, 2048
    k, v = mixture(b, h, t, seed=11), mixture(b, h, t, seed=12)
    q = gaussian(b, 32, 1, 128, seed=13)
    cache = compress(cuda(k), cuda(v), ResKVKernelConfig(sparsity=0.5, bits=16))
    out = attention(cuda(q), cache, position=t)
    assert_attention_close(out, reference(q, cache, position=t))
    dense = oatt.attention_dense(np16(q), np16(k).astype(np.float32), np16(v).astype(np.float32), position=t)
    rel = np.linalg.norm(out.float().cpu().numpy() - dense) / np.linalg.norm(dense)
    assert rel < 0.15, rel

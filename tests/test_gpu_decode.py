"""CUDA decode attention (unstructured FP16 bitmap layout) against the oracle
and against vectors recorded from the reference's own FP32 attention."""

import numpy as np
import pytest
import torch

from helpers import assert_attention_close, np16, oracle_attention, oracle_cache, to_compressed
from oracle import attention as oatt

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True, params=["tensor-core", "simt"])
def kernel_variant(request):
    """Every test runs against both partial kernels."""
    from reskv_b200._extension import library

    lib = library()
    assert lib.reskv_decode_set_variant(0 if request.param == "tensor-core" else 1) == 0
    yield request.param
    lib.reskv_decode_set_variant(0)


def _plan(nnz):
    from reskv_b200.config import KernelPlan

    return KernelPlan("unstructured", "deferred", 16, nnz, 2, 0)


def _case(b, kh, gqa, t, nnz, ck=32, cv=32, seed=0):
    from reskv_b200.synthetic import gaussian, mixture

    k = mixture(b, kh, t, seed=seed)
    v = mixture(b, kh, t, seed=seed + 1)
    q = gaussian(b, kh * gqa, 1, 128, seed=seed + 2)
    kc = gaussian(b, kh, ck, 128, seed=seed + 3)
    vc = gaussian(b, kh, cv, 128, seed=seed + 4)
    g = torch.Generator().manual_seed(seed + 5)
    ki = torch.randint(ck, (b, kh, t), generator=g, dtype=torch.int32)
    vi = torch.randint(cv, (b, kh, t), generator=g, dtype=torch.int32)
    kcache = oracle_cache(k, kc, ki, "unstructured", 16, nnz)
    vcache = oracle_cache(v, vc, vi, "unstructured", 16, nnz)
    return q, kcache, vcache


def _run(q, kcache, vcache, nnz, **kw):
    from reskv_b200 import attention
    from reskv_b200.tensors import CompressedKV

    cache = CompressedKV(to_compressed(kcache, _plan(nnz), DEV), to_compressed(vcache, _plan(nnz), DEV))
    kw = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in kw.items()}
    if kw.get("recent") is not None:
        kw["recent"] = tuple(r.to(DEV) for r in kw["recent"])
    return attention(q.to(DEV), cache, **kw)


@pytest.mark.parametrize("nnz", [32, 64])
@pytest.mark.parametrize("t", [1, 63, 64, 65, 200, 1000, 2500])
def test_matches_oracle_over_lengths(t, nnz):
    q, kc, vc = _case(2, 2, 4, t, nnz, seed=t)
    out = _run(q, kc, vc, nnz, position=t + 3)
    assert_attention_close(out, oracle_attention(q, kc, vc, position=t + 3))


def test_reference_cpu_configuration_at_full_size():
    """One sequence of 8 KV heads at context 8192 as the reference's CPU case sets it up: 4 sink
    tokens kept dense (start_position = 4), 8128 compressed tokens at sparsity 0.5, the remaining 60
    tokens plus the sinks in the dense segment."""
    t, sinks, dense = 8128, 4, 60
    q, kc, vc = _case(1, 8, 4, t, 64, seed=21)
    pos = sinks + t + dense - 1
    freq = (500000.0 ** (-torch.arange(64).float() / 64)).float()
    qr = torch.from_numpy(oatt.rotate(np16(q), np.array([pos]), np16(freq))).half()
    g = torch.Generator().manual_seed(22)
    kr = (torch.randn(1, 8, sinks + dense, 128, generator=g) * 0.5).half()  # rotated sink + window keys
    vr = (torch.randn(1, 8, sinks + dense, 128, generator=g) * 0.5).half()
    kw = dict(position=pos, start_position=sinks, recent=(qr, kr, vr))
    out = _run(q, kc, vc, 64, **kw)
    assert_attention_close(out, oracle_attention(q, kc, vc, **kw))


@pytest.mark.parametrize("nnz", [32, 64])
def test_long_context_head(nnz):
    """65 472 compressed tokens (the 64K-context case): positions far from the query, 1023 tiles,
    split-K over many CTAs."""
    t = 65472
    q, kc, vc = _case(1, 1, 4, t, nnz, seed=31 + nnz)
    out = _run(q, kc, vc, nnz, position=t + 63)
    assert_attention_close(out, oracle_attention(q, kc, vc, position=t + 63))


@pytest.mark.parametrize("gqa", [1, 4, 8])
@pytest.mark.parametrize("clusters", [1, 32, 33, 64])
def test_head_ratios_and_centroid_counts(gqa, clusters):
    q, kc, vc = _case(1, 3, gqa, 320, 32, ck=clusters, cv=clusters, seed=gqa * 100 + clusters)
    out = _run(q, kc, vc, 32, position=330, start_position=10)
    assert_attention_close(out, oracle_attention(q, kc, vc, position=330, start_position=10))


def test_model_frequencies_scaling_and_recent_window():
    t = 700
    q, kc, vc = _case(2, 2, 4, t, 32, seed=7)
    freq = (500000.0 ** (-torch.arange(64).float() / 64) / torch.linspace(1, 8, 64)).float()
    qr = torch.from_numpy(oatt.rotate(np16(q), np.array([t + 40]), np16(freq))).half()
    g = torch.Generator().manual_seed(3)
    kr = (torch.randn(2, 2, 33, 128, generator=g) * 0.5).half()
    vr = (torch.randn(2, 2, 33, 128, generator=g) * 0.5).half()
    kw = dict(position=t + 40, inv_freq=freq, scaling=0.11, recent=(qr, kr, vr))
    out = _run(q, kc, vc, 32, **kw)
    assert_attention_close(out, oracle_attention(q, kc, vc, **kw))


@pytest.mark.parametrize("splits", [1, 3, 7, 64])
def test_split_count_does_not_change_the_result(splits):
    from reskv_b200.config import KernelPlan

    t = 1500
    q, kc, vc = _case(1, 2, 4, t, 32, seed=11)
    from reskv_b200 import attention
    from reskv_b200.tensors import CompressedKV

    plan = KernelPlan("unstructured", "deferred", 16, 32, 2, splits)
    cache = CompressedKV(to_compressed(kc, plan, DEV), to_compressed(vc, plan, DEV))
    out = attention(q.to(DEV), cache, position=t)
    assert_attention_close(out, oracle_attention(q, kc, vc, position=t))


def test_stats_and_separate_recent_merge_match_the_fused_call():
    """decode_fp16 -> (out, m, l) then merge_recent, the reference's two-step
    form (reskv/_attention.py:59-76,117-143), equals the fused call."""
    from reskv_b200._extension import load_extension

    t = 900
    q, kc, vc = _case(2, 2, 4, t, 64, seed=21)
    plan = _plan(64)
    k, v = to_compressed(kc, plan, DEV), to_compressed(vc, plan, DEV)
    ext = load_extension("cluster_mass", plan, 0)
    qf = q.to(DEV).reshape(-1, 128)
    args = (qf, *k._native[:4], *v._native[:4], 2, 8, 0, t + 5, 500000.0, 128**-0.5)
    out, m, l = ext.decode_fp16(*args, True, 0, None)
    dense_k = oatt.layouts.reconstruct(**kc)
    dense_v = oatt.layouts.reconstruct(**vc)
    want, wm, wl = oatt.attention_dense(np16(q), dense_k, dense_v, position=t + 5, return_stats=True)
    assert_attention_close(out, want)
    np.testing.assert_allclose(m.cpu().numpy().reshape(wm.shape), wm, atol=2e-3, rtol=1e-4)
    np.testing.assert_allclose(l.cpu().numpy().reshape(wl.shape), wl, rtol=5e-3)
    g = torch.Generator().manual_seed(5)
    qr = torch.randn(2, 8, 1, 128, generator=g).half()
    kr = torch.randn(2, 2, 40, 128, generator=g).half()
    vr = torch.randn(2, 2, 40, 128, generator=g).half()
    want = oatt.attention_dense(np16(q), dense_k, dense_v, position=t + 5, recent=(np16(qr), np16(kr), np16(vr)))
    scores = torch.einsum("bhgd,bhtd->bhgt", qr.float().reshape(2, 2, 4, 128), kr.float()) * 128**-0.5
    scores = scores.reshape(2, 8, 40).contiguous().to(DEV)
    merged = ext.merge_recent(out, m, l, scores, vr.to(DEV), 2, 8)
    assert_attention_close(merged, want)
    att = load_extension("attention", plan, 0)
    merged2 = att.merge_recent(out, m, l, qr.to(DEV).reshape(-1, 128), kr.to(DEV), vr.to(DEV), 2, 8, 128**-0.5)
    assert_attention_close(merged2, want)
    (fused,) = ext.decode_fp16(*args, False, 0, None, (qr.to(DEV).reshape(-1, 128), kr.to(DEV), vr.to(DEV)))
    assert_attention_close(fused, want)


@pytest.mark.parametrize("nnz", [32, 64])
def test_large_finite_recent_scores(nnz):
    """Zero cache, recent logits of 1e5: the joint softmax must stay finite
    (reference tests/test_cuda.py:146-158)."""
    from reskv_b200 import ResKVKernelConfig, attention
    from reskv_b200.tensors import CompressedKV

    data = torch.zeros(1, 1, 128, 128, dtype=torch.float16)
    cen = data[:, :, :1].contiguous()
    ids = torch.zeros(1, 1, 128, dtype=torch.int32)
    kc = oracle_cache(data, cen, ids, "unstructured", 16, nnz)
    plan = ResKVKernelConfig(sparsity=1 - nnz / 128, layout="unstructured").resolve(1)
    cache = CompressedKV(to_compressed(kc, plan, DEV), to_compressed(kc, plan, DEV))
    query = torch.full((1, 4, 1, 128), 100.0, dtype=torch.float16)
    recent = (query, torch.full((1, 1, 32, 128), 100.0, dtype=torch.float16),
              torch.full((1, 1, 32, 128), 2.0, dtype=torch.float16))
    out = attention(query.to(DEV), cache, position=159, recent=tuple(r.to(DEV) for r in recent))
    want = oracle_attention(query, kc, kc, position=159, recent=recent)
    assert torch.isfinite(out).all()
    assert_attention_close(out, want, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("nnz", [32, 64])
def test_against_vectors_recorded_from_the_reference(golden, nnz):
    """Caches encoded by the reference's own ``_encode`` and outputs of its own
    ``reference_attention`` (tests/golden/make_golden.py)."""
    g = golden
    t = g["x_k"].shape[2]

    def cache(tag, flavour):
        cen, ids = (g["cen_k"], g["ids_k"]) if tag == "k" else (g["cen_v"], g["ids_v"])
        return dict(layout="unstructured", bits=16, centroids=cen, ids=ids,
                    payload=g[f"enc_u16_{tag}_{nnz}_{flavour}_payload"],
                    metadata=g[f"enc_u16_{tag}_{nnz}_{flavour}_meta"], scale=None)

    k, v = cache("k", "k"), cache("v", "v")
    q = torch.from_numpy(g["q"])
    freq = torch.from_numpy(g["freq_model"])
    assert_attention_close(_run(q, k, v, nnz, position=t + 40), g[f"att_{nnz}_theta"])
    out = _run(q, k, v, nnz, position=t + 40, start_position=7, inv_freq=freq, scaling=0.11)
    assert_attention_close(out, g[f"att_{nnz}_freq_start"])
    rec = tuple(torch.from_numpy(g[f"att_{nnz}_{n}"]) for n in ("qr", "kr", "vr"))
    out = _run(q, k, v, nnz, position=t + 40, inv_freq=freq, recent=rec)
    assert_attention_close(out, g[f"att_{nnz}_recent"])


def test_capacity_windows_and_append_are_read_in_place():
    """Tensors that are windows of larger buffers (token stride > tokens)."""
    t, add = 300, 64
    q, kc, vc = _case(2, 2, 4, t + add, 32, seed=31)
    from reskv_b200 import attention
    from reskv_b200.tensors import CompressedKV, CompressedTensor

    plan = _plan(32)

    def split(c, lo, hi):
        d = dict(c)
        for key in ("ids", "payload", "metadata"):
            d[key] = c[key][:, :, lo:hi]
        return d

    k = to_compressed(split(kc, 0, t), plan, DEV).append(to_compressed(split(kc, t, t + add), plan, DEV))
    v = to_compressed(split(vc, 0, t), plan, DEV).append(to_compressed(split(vc, t, t + add), plan, DEV))
    assert k.token_stride > k.seq_len == t + add
    out = attention(q.to(DEV), CompressedKV(k, v), position=t + add)
    assert_attention_close(out, oracle_attention(q, kc, vc, position=t + add))


def test_argument_errors():
    from reskv_b200 import attention
    from reskv_b200.tensors import CompressedKV

    q, kc, vc = _case(1, 1, 4, 64, 32, seed=41)
    cache = CompressedKV(to_compressed(kc, _plan(32), DEV), to_compressed(vc, _plan(32), DEV))
    with pytest.raises(ValueError, match="precedes"):
        attention(q.to(DEV), cache, position=10)
    with pytest.raises(ValueError, match="query must be FP16 CUDA"):
        attention(q.to(DEV).float(), cache, position=64)
    with pytest.raises(ValueError, match="ratios"):
        attention(q.to(DEV)[:, :2].contiguous(), cache, position=64)

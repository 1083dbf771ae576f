"""This library against outputs recorded from the reference's own CUDA code on a B200
(``tests/golden/reference_gpu_vectors.npz``, written by ``tests/golden/make_golden_gpu.py``):
packers bit-exact, V-path clustering, the eleven attention plans, and a full-size
quantised case (16 320 tokens, theta 1e6) pinned by digests of the reference's packed words."""

import hashlib

import numpy as np
import pytest
import torch

from helpers import ATOL, RTOL, np16
from oracle import encode as oenc
from oracle import kmeans as okm

from golden.make_golden_gpu import CASES, PACKER_PLANS, case_tag

pytestmark = pytest.mark.gpu
DEV = "cuda"


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _plan(layout, bits, nnz):
    from reskv_b200.config import KernelPlan

    fusion = {"unstructured": "deferred" if bits == 16 else "per_token", "tiled": "per_token", "structured": "deferred"}[layout]
    return KernelPlan(layout, fusion, bits, nnz, 4, 0)


def _bits(a):
    return a.view(np.uint16) if a.dtype == np.float16 else a


@pytest.mark.parametrize("layout,bits,nnz", PACKER_PLANS)
def test_packers_reproduce_the_reference_kernels_bit_for_bit(gpu_golden, layout, bits, nnz):
    from reskv_b200.compression import _encode

    g = gpu_golden
    ct = _encode(T(g["pk_x"]), T(g["pk_cen"]), T(g["pk_ids"]), _plan(layout, bits, nnz))
    key = f"pk_{layout}_{bits}_{nnz}"
    assert np.array_equal(_bits(np16(ct.payload)), _bits(g[key + "_payload"]))
    if ct.metadata is not None:
        assert np.array_equal(np16(ct.metadata), g[key + "_meta"])
    if ct.scale is not None:
        assert np.array_equal(_bits(np16(ct.scale)), _bits(g[key + "_scale"]))


@pytest.mark.parametrize("nnz", [32, 64])
def test_bitmap_encoder_against_the_reference_torch_path_on_the_device(gpu_golden, nnz):
    from reskv_b200.compression import _encode

    g = gpu_golden
    ct = _encode(T(g["pk_x"]), T(g["pk_cen"]), T(g["pk_ids"]), _plan("unstructured", 16, nnz))
    keys = np.abs(oenc.residual_fp32(g["pk_x"], g["pk_cen"], g["pk_ids"]).astype(np.float16)).astype(np.float32)
    ties = oenc.tie_tokens(keys, nnz)
    for flavour in ("k", "v"):
        key = f"pk_unstructured_16_{nnz}_{flavour}"
        assert np.array_equal(np16(ct.metadata)[~ties], g[key + "_meta"][~ties])
        assert np.array_equal(_bits(np16(ct.payload))[~ties], _bits(g[key + "_payload"])[~ties])


@pytest.mark.parametrize("value", [0, 1])
@pytest.mark.parametrize("count,iters", [(8, 1), (8, 4), (32, 3), (32, 10)])
def test_clustering_against_the_reference_on_the_device(gpu_golden, value, count, iters):
    """Ids equal the reference's outside near-ties (its matrix-form distances, FP16 for V, may pick the
    other centre there); with equal ids the centres are equal to the bit for a single step."""
    from reskv_b200.compression import cluster

    g = gpu_golden
    cen, ids = cluster(T(g["km_x"]), count, iters, value=bool(value))
    ref_c, ref_i = g[f"km_{value}_{count}_{iters}_centres"], g[f"km_{value}_{count}_{iters}_ids"]
    differ = np16(ids) != ref_i
    if iters == 1:
        _, _, margin = okm.cluster(g["km_x"], count, 1, value=bool(value))
        assert not (differ & (margin > (2e-2 if value else 1e-4))).any()
        if not differ.any():
            assert np.array_equal(_bits(np16(cen)), _bits(ref_c))
    assert differ.mean() <= (0.06 if value else 0.005)


def test_value_cluster_mean_does_not_overflow(gpu_golden):
    from reskv_b200.compression import cluster

    data = torch.full((1, 1, 8192, 128), 20.0, device=DEV, dtype=torch.float16)
    for count in (1, 32):
        cen, ids = cluster(data, count=count, iterations=2, value=True)
        assert np.array_equal(np16(ids), gpu_golden[f"km_const_{count}_ids"])
        restored = cen.gather(2, ids.long().unsqueeze(-1).expand_as(data))
        assert torch.equal(restored, data)


def _tensor(g, tag, side, plan):
    from reskv_b200.tensors import CompressedTensor

    meta, scale = g.get(f"{tag}_{side}_meta"), g.get(f"{tag}_{side}_scale")
    return CompressedTensor(T(g[f"at_{side}c"]), T(g[f"at_{side}i"]), T(g[f"{tag}_{side}_payload"]),
                            None if meta is None else T(meta), None if scale is None else T(scale), plan)


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("bits,sparsity,layout,fusion", CASES)
def test_attention_on_the_reference_packed_caches(gpu_golden, bits, sparsity, layout, fusion, variant):
    """The caches the reference's ``compress`` produced, fed to this library's ``attention``: within
    |a - b| <= 2e-3 + 1e-2 |b| of the reference's FP32 attention, with and without the recent window."""
    from reskv_b200 import ResKVKernelConfig, attention, compress
    from reskv_b200._extension import library
    from reskv_b200.tensors import CompressedKV

    g = gpu_golden
    tag = "at_" + case_tag(bits, sparsity, layout, fusion)
    cfg = ResKVKernelConfig(bits=bits, sparsity=sparsity, layout=layout, centroid_fusion=fusion)
    plan = cfg.resolve(1)
    cache = CompressedKV(_tensor(g, tag, "k", plan), _tensor(g, tag, "v", plan))
    lib = library()
    assert lib.reskv_decode_set_variant(variant) == 0
    try:
        for suffix, recent in (("", None), ("_recent", (T(g["at_qr"]), T(g["at_kr"]), T(g["at_vr"])))):
            out = attention(T(g["at_q"]), cache, position=288, inv_freq=T(g["at_freq"]), recent=recent)
            want = g[tag + "_ref" + suffix]
            err = np.abs(np16(out.float()) - want)
            assert (err <= ATOL + RTOL * np.abs(want)).all(), f"max err {err.max():.3e}"
    finally:
        lib.reskv_decode_set_variant(0)
    # and this library's own compress() reproduces the reference's packed tensors (ties of the torch encoder aside)
    mine = compress(T(g["at_k"]), T(g["at_v"]), cfg, clustering=((T(g["at_kc"]), T(g["at_ki"])), (T(g["at_vc"]), T(g["at_vi"]))))
    if not (bits == 16 and layout == "unstructured"):
        for got, side in ((mine.key, "k"), (mine.value, "v")):
            assert np.array_equal(_bits(np16(got.payload)), _bits(g[f"{tag}_{side}_payload"]))
            if got.scale is not None:
                assert np.array_equal(_bits(np16(got.scale)), _bits(g[f"{tag}_{side}_scale"]))
            if got.metadata is not None:
                assert np.array_equal(np16(got.metadata), g[f"{tag}_{side}_meta"])


def _digest(t):
    return np.frombuffer(hashlib.sha256(t.detach().cpu().contiguous().numpy().tobytes()).digest(), np.uint8)


@pytest.mark.parametrize("bits", [4, 2, 16])
def test_full_size_context_16384(gpu_golden, bits):
    """Qwen3-8B layer shape (same head geometry), context 16 384 -> 16 320 compressed tokens, theta 1e6,
    sparsity 0.5 with INT4 / INT2 residuals: packed words and scales equal the reference kernel's
    (SHA-256 of the whole tensor), attention within tolerance of its FP32 attention.  bits 16: the FP16
    bitmap layout at sparsity 0.75 and theta 5e5 on the same inputs."""
    from reskv_b200 import ResKVKernelConfig, attention, compress
    from reskv_b200.synthetic import mixture

    g = gpu_golden
    fb, fh, ft, seed = (int(x) for x in g["fs_shape"])
    k, v = mixture(fb, fh, ft, seed=seed), mixture(fb, fh, ft, seed=seed + 1)
    if not (np.array_equal(_digest(k), g["fs_k_digest"]) and np.array_equal(_digest(v), g["fs_v_digest"])):
        pytest.skip("the CPU generator of this torch build draws other inputs than the recorded run used")
    clustering = ((T(g["fs_kc"]), T(g["fs_ki"].astype(np.int32))), (T(g["fs_vc"]), T(g["fs_vi"].astype(np.int32))))
    q = T(g["fs_q"])
    if bits == 16:
        cache = compress(k.to(DEV), v.to(DEV), ResKVKernelConfig(bits=16, sparsity=0.75, layout="unstructured"), clustering=clustering)
        out, want = attention(q, cache, position=16384), g["fs_fp16_ref"]
    else:
        cache = compress(k.to(DEV), v.to(DEV), ResKVKernelConfig(bits=bits, sparsity=0.5, layout="unstructured"), clustering=clustering)
        tag = f"fs_int{bits}"
        assert np.array_equal(_digest(cache.key.payload), g[tag + "_k_payload_digest"])
        assert np.array_equal(_digest(cache.key.scale), g[tag + "_k_scale_digest"])
        assert np.array_equal(_digest(cache.value.payload), g[tag + "_v_payload_digest"])
        assert np.array_equal(_digest(cache.value.scale), g[tag + "_v_scale_digest"])
        out, want = attention(q, cache, position=16384, inv_freq=T(g["fs_freq"])), g[tag + "_ref"]
    err = np.abs(np16(out.float()) - want)
    assert (err <= ATOL + RTOL * np.abs(want)).all(), f"max err {err.max():.3e}"

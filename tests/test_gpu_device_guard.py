"""Calls made while another GPU is the current device (needs two GPUs; skipped on one).

The reference's ops switch to their tensors' device (``CUDAGuard``, reskv/csrc/cluster_mass.cu:1187,
attention.cu:684, compression.cu:396).  Here the Python operator tables make the tensors' device
current around every library call, and the C entry points refuse memory of another device."""

import pytest
import torch

from helpers import assert_attention_close, np16, oracle_attention

pytestmark = pytest.mark.gpu


def _two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")


def _as_oracle(ct):
    p = ct.plan
    return dict(layout=p.layout, bits=p.bits, centroids=np16(ct.centroids), ids=np16(ct.cluster_ids),
                payload=np16(ct.payload), metadata=None if ct.metadata is None else np16(ct.metadata),
                scale=None if ct.scale is None else np16(ct.scale))


@pytest.mark.parametrize("bits", [16, 4])
def test_cache_on_the_second_gpu_while_the_first_is_current(bits):
    _two_gpus()
    from reskv_b200 import ResKVKernelConfig, attention, compress
    from reskv_b200.compression import cluster
    from reskv_b200.synthetic import gaussian, mixture

    torch.cuda.set_device(0)
    other = torch.device("cuda", 1)
    b, h, t = 1, 2, 300
    k, v = mixture(b, h, t, seed=11), mixture(b, h, t, seed=12)
    q = gaussian(b, h * 4, 1, 128, seed=13)
    cfg = ResKVKernelConfig(bits=bits, sparsity=0.5, layout="unstructured", num_clusters=8, kmeans_iterations=3)
    cache = compress(k.to(other), v.to(other), cfg)          # k-means + packers on cuda:1
    out = attention(q.to(other), cache, position=t + 5)       # decode + merge on cuda:1
    torch.cuda.synchronize(other)
    assert torch.cuda.current_device() == 0
    assert out.device == other and cache.key.payload.device == other
    want = oracle_attention(q, _as_oracle(cache.key), _as_oracle(cache.value), position=t + 5)
    assert_attention_close(out, want)
    centres, ids = cluster(k.to(other), 8, 2)
    assert centres.device == other and ids.device == other


def test_raw_call_with_the_other_gpus_memory_is_refused():
    _two_gpus()
    from reskv_b200._extension import ERR_INVALID, library

    lib = library()
    torch.cuda.set_device(0)
    other = torch.device("cuda", 1)
    t = 64
    x = torch.zeros(1, 1, t, 128, dtype=torch.float16, device=other)
    cen = torch.zeros(1, 1, 4, 128, dtype=torch.float16, device=other)
    ids = torch.zeros(1, 1, t, dtype=torch.int32, device=other)
    pay = torch.empty(1, 1, t, 32, dtype=torch.float16, device=other)
    bm = torch.empty(1, 1, t, 2, dtype=torch.int64, device=other)
    rc = lib.reskv_encode_bitmap_fp16(x.data_ptr(), cen.data_ptr(), ids.data_ptr(), 1, 1, t, t, 4, 32, pay.data_ptr(),
                                      bm.data_ptr(), t, torch.cuda.current_stream(0).cuda_stream)
    assert rc == ERR_INVALID
    msg = lib.reskv_last_error().decode()
    assert "lives on device 1" in msg and "device 0 is current" in msg


def test_tensors_of_two_devices_in_one_call_are_refused():
    _two_gpus()
    from reskv_b200 import ResKVKernelConfig, attention, compress
    from reskv_b200.synthetic import gaussian, mixture

    k = mixture(1, 1, 128, seed=1)
    cfg = ResKVKernelConfig(num_clusters=4, kmeans_iterations=1)
    cache = compress(k.to("cuda:1"), k.to("cuda:1"), cfg)
    with pytest.raises(ValueError, match="same CUDA device"):
        attention(gaussian(1, 4, 1, 128, seed=2).to("cuda:0"), cache, position=200)

"""Compact quantised layout (bitmap + codes of the retained coordinates): oracle
round trip, plan rules and tensor shapes.  CPU only."""

import numpy as np
import pytest

from oracle import encode as oenc
from oracle import layouts as olay


@pytest.mark.parametrize("bits,nnz", [(4, 64), (4, 32), (2, 64)])
def test_oracle_compact_equals_quantised(bits, nnz):
    rng = np.random.default_rng(bits * 100 + nnz)
    x = (rng.standard_normal((2, 3, 70, 128)) * np.exp(rng.standard_normal(128))).astype(np.float16)
    cen = rng.standard_normal((2, 3, 9, 128)).astype(np.float16)
    ids = rng.integers(0, 9, (2, 3, 70))
    words, bitmap, scale = oenc.encode("compact", bits, nnz, x, cen, ids)
    full, none, scale_q = oenc.encode("unstructured", bits, nnz, x, cen, ids)
    assert none is None and np.array_equal(scale, scale_q)
    assert words.shape[-1] == nnz * bits // 32 and bitmap.shape[-1] == 2
    assert olay.mask_unstructured_fp16(bitmap).sum(-1).max() == nnz
    a = olay.reconstruct("compact", bits, cen, ids, words, bitmap, scale)
    b = olay.reconstruct("unstructured", bits, cen, ids, full, None, scale_q)
    assert np.array_equal(a, b)


def test_plan_rules():
    from reskv_b200 import ResKVKernelConfig
    from reskv_b200.config import KernelPlan

    plan = ResKVKernelConfig(bits=4, sparsity=0.5, layout="compact").resolve(8)
    assert (plan.layout, plan.centroid_fusion, plan.bits, plan.nnz) == ("compact", "per_token", 4, 64)
    assert ResKVKernelConfig(bits=4, sparsity=0.75, layout="compact").resolve(1).nnz == 32
    assert ResKVKernelConfig(bits=2, sparsity=0.5, layout="compact").resolve(1).nnz == 64
    for bad in (dict(bits=16, sparsity=0.5), dict(bits=2, sparsity=0.75)):
        with pytest.raises(ValueError, match="compact layout"):
            ResKVKernelConfig(layout="compact", **bad)
    with pytest.raises(ValueError, match="per_token"):
        ResKVKernelConfig(bits=4, layout="compact", centroid_fusion="deferred").resolve(1)
    with pytest.raises(ValueError, match="compact"):
        KernelPlan("compact", "per_token", 2, 32, 4, 0)
    # the reference's own choices are untouched: "auto" never picks the compact layout
    for sparsity in (0.5, 0.75):
        for bits in (2, 4, 16):
            assert ResKVKernelConfig(bits=bits, sparsity=sparsity).resolve(4).layout != "compact"


def test_tensor_shapes():
    import torch

    from reskv_b200.config import KernelPlan
    from reskv_b200.tensors import CompressedTensor, metadata_spec, payload_width

    plan = KernelPlan("compact", "per_token", 4, 64, 4, 0)
    assert payload_width(plan) == 8 and metadata_spec(plan) == (2, torch.int64)
    cen = torch.zeros(1, 1, 4, 128, dtype=torch.float16)
    ids = torch.zeros(1, 1, 5, dtype=torch.int32)
    ok = CompressedTensor(cen, ids, torch.zeros(1, 1, 5, 8, dtype=torch.int32), torch.zeros(1, 1, 5, 2, dtype=torch.int64),
                          torch.ones(1, 1, 5, dtype=torch.float16), plan)
    assert ok.seq_len == 5
    with pytest.raises(ValueError, match="payload width"):
        CompressedTensor(cen, ids, torch.zeros(1, 1, 5, 16, dtype=torch.int32), torch.zeros(1, 1, 5, 2, dtype=torch.int64),
                         torch.ones(1, 1, 5, dtype=torch.float16), plan)
    with pytest.raises(ValueError, match="scales"):
        CompressedTensor(cen, ids, torch.zeros(1, 1, 5, 8, dtype=torch.int32), torch.zeros(1, 1, 5, 2, dtype=torch.int64),
                         None, plan)

"""The allocation-free decode entry point (``reskv_decode_bitmap_fp16_noalloc``).

Some hosts of this library cannot hand it scratch memory at the call site: a
serving process whose memory pool owns the whole device, a plug-in called from a
loop where an allocation would stall the GPU, a C or cgo host without torch's
allocator.  For them the library keeps the split-K scratch of the decode call in
a fixed 8 MiB array of its own.  This test drives that entry point directly
through the C ABI, twice in a row (the second call finds the first call's data
in the shared array), and compares with the workspace-taking entry point; it
also checks that an over-sized problem is refused with a message instead of
overrunning the array.

Collected last on purpose (file name), and independent of the other tests: it
passes in a fresh process as well as after the rest of the suite.
"""

import ctypes

import numpy as np
import pytest
import torch

from helpers import ATOL, RTOL, oracle_attention, oracle_cache, to_compressed

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(b, kh, gqa, t, nnz, seed):
    from reskv_b200.config import KernelPlan
    from reskv_b200.synthetic import gaussian, mixture

    k, v = mixture(b, kh, t, seed=seed), mixture(b, kh, t, seed=seed + 1)
    q = gaussian(b, kh * gqa, 1, 128, seed=seed + 2)
    cen = gaussian(b, kh, 32, 128, seed=seed + 3)
    ids = torch.randint(32, (b, kh, t), generator=torch.Generator().manual_seed(seed), dtype=torch.int32)
    kc = oracle_cache(k, cen, ids, "unstructured", 16, nnz)
    vc = oracle_cache(v, cen, ids, "unstructured", 16, nnz)
    plan = KernelPlan("unstructured", "deferred", 16, nnz, 2, 0)
    return q, kc, vc, to_compressed(kc, plan, DEV), to_compressed(vc, plan, DEV)


def _call_noalloc(lib, q, key, value, kh, nh, pos, splits, recent=None):
    kcen, ki, kp, km, _ = key._native
    vcen, vi, vp, vm, _ = value._native
    bnh = q.shape[0]
    out = torch.empty((bnh, 128), dtype=torch.float16, device=DEV)
    m = torch.empty(bnh, dtype=torch.float32, device=DEV)
    l = torch.empty(bnh, dtype=torch.float32, device=DEV)
    rq, rk, rv, tr = None, None, None, 0
    if recent is not None:
        rq, rk, rv = (x.data_ptr() for x in recent)
        tr = recent[1].shape[2]
    rc = lib.reskv_decode_bitmap_fp16_noalloc(
        q.data_ptr(), kcen.data_ptr(), ki.data_ptr(), kp.data_ptr(), km.data_ptr(), vcen.data_ptr(), vi.data_ptr(),
        vp.data_ptr(), vm.data_ptr(), bnh // nh, kh, nh, kp.shape[1], key.token_stride, kcen.shape[1], vcen.shape[1],
        kp.shape[2], 0, pos, 500000.0, None, 128**-0.5, splits, rq, rk, rv, tr, out.data_ptr(), m.data_ptr(),
        l.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, out, m, l


def _close(a, b):
    a, b = a.float().cpu().numpy(), b.float().cpu().numpy()
    return (np.abs(a - b) <= ATOL + RTOL * np.abs(b)).all()


@pytest.mark.parametrize("nnz", [32, 64])
def test_matches_the_workspace_entry_point_on_consecutive_calls(nnz):
    from reskv_b200._extension import library, load_extension

    lib = library()
    b, kh, gqa, t = 2, 2, 4, 1500
    q, kc, vc, key, value = _case(b, kh, gqa, t, nnz, seed=70 + nnz)
    qd = q.to(DEV).reshape(-1, 128)
    ops = load_extension("cluster_mass", key.plan, 0)
    ref, ref_m, ref_l = ops.decode_fp16(qd, *key._native[:4], *value._native[:4], kh, kh * gqa, 0, t + 2, 500000.0,
                                        128**-0.5, True, 0, None)
    g = torch.Generator().manual_seed(1)
    recent = tuple(x.to(DEV) for x in (torch.randn(b * kh * gqa, 128, generator=g).half(),
                                       torch.randn(b, kh, 20, 128, generator=g).half(),
                                       torch.randn(b, kh, 20, 128, generator=g).half()))
    (ref_recent,) = ops.decode_fp16(qd, *key._native[:4], *value._native[:4], kh, kh * gqa, 0, t + 2, 500000.0,
                                    128**-0.5, False, 0, None, recent)
    # first call, then a different problem (other split count, recent window) that reuses the
    # same built-in scratch, then the first problem again
    for splits, rec, want in ((0, None, ref), (5, recent, ref_recent), (0, None, ref)):
        rc, out, m, l = _call_noalloc(lib, qd, key, value, kh, kh * gqa, t + 2, splits, rec)
        assert rc == 0, lib.reskv_last_error().decode()
        # no bounded wait ran out and no slot index was out of range: the status word of the built-in scratch is 0
        status = torch.full((1,), 0xFFFF, dtype=torch.int32).pin_memory()
        assert lib.reskv_decode_noalloc_status(status.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert _close(out, want)
        if rec is None:
            assert torch.allclose(m, ref_m, atol=2e-3) and torch.allclose(l, ref_l, rtol=5e-3)
    # and against the CPU oracle, so that both entry points being wrong together would show
    want = oracle_attention(q, kc, vc, position=t + 2)
    assert _close(out.reshape(want.shape), torch.from_numpy(want))


def test_problem_beyond_the_builtin_scratch_is_refused():
    from reskv_b200._extension import library

    lib = library()
    b, kh, gqa, t = 16, 8, 8, 1024  # 1024 query heads x 16 splits x 776 B > 8 MiB
    q, _, _, key, value = _case(b, kh, gqa, t, 32, seed=5)
    rc, *_ = _call_noalloc(lib, q.to(DEV).reshape(-1, 128), key, value, kh, kh * gqa, t, 16)
    assert rc == -4
    msg = lib.reskv_last_error().decode()
    assert "built-in" in msg and "splits" in msg
    # the same problem with fewer splits fits and runs
    rc, out, *_ = _call_noalloc(lib, q.to(DEV).reshape(-1, 128), key, value, kh, kh * gqa, t, 4)
    assert rc == 0, lib.reskv_last_error().decode()
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()

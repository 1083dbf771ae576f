"""Decode driven by a device-side step state (the entry points a CUDA-graph decode
loop uses): results must equal the by-value ``attention()`` call for the same cache,
whether the compressed token count comes from the launch arguments or from the state."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
PLANS = [(0.75, 16, "unstructured"), (0.5, 16, "unstructured"), (0.5, 16, "tiled"), (0.75, 16, "structured"),
         (0.5, 4, "unstructured"), (0.5, 2, "unstructured"), (0.75, 4, "structured")]


@pytest.fixture(autouse=True, params=["tensor-core", "simt"])
def kernel_variant(request):
    from reskv_b200._extension import library

    lib = library()
    assert lib.reskv_decode_set_variant(0 if request.param == "tensor-core" else 1) == 0
    yield request.param
    lib.reskv_decode_set_variant(0)


def _rope(x, pos, inv_freq):
    ang = float(pos) * inv_freq
    cos, sin = torch.cos(ang), torch.sin(ang)
    a, b = x.float()[..., :64], x.float()[..., 64:]
    return torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1).to(x.dtype)


def _step(cache, q, qr, win_k, win_v, state, tokens_arg, splits, rows=None):
    """One reskv_decode_step call; centroid tables optionally padded to `rows` zero rows."""
    from reskv_b200 import _extension as ext

    lib = ext.library()
    key, val = cache.key, cache.value
    plan = key.plan
    kc, ki, kp, km, ks = key._native
    vc, vi, vp, vm, vs = val._native
    if rows is not None:
        pad_k = torch.zeros((kc.shape[0], rows, 128), dtype=torch.float16, device=DEV)
        pad_v = torch.zeros_like(pad_k)
        pad_k[:, :kc.shape[1]] = kc
        pad_v[:, :vc.shape[1]] = vc
        kc, vc = pad_k, pad_v
    b, hq = q.shape[:2]
    hkv = key.centroids.shape[1]
    layout = {"unstructured": ext.LAYOUT_UNSTRUCTURED, "tiled": ext.LAYOUT_TILED, "structured": ext.LAYOUT_STRUCTURED}[plan.layout]
    need = lib.reskv_decode_bitmap_fp16_workspace_bytes(b, hkv, hq, 1 << 16, 64)
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    out = torch.empty((b * hq, 128), dtype=torch.float16, device=DEV)
    inv = (500000.0 ** (-torch.arange(64, device=DEV).float() / 64)).contiguous()

    def ptr(t):
        return None if t is None else t.data_ptr()

    qf, qrf = q.reshape(b * hq, 128).contiguous(), qr.reshape(b * hq, 128).contiguous()
    rc = lib.reskv_decode_step(layout, plan.bits, kp.shape[2], qf.data_ptr(), kc.data_ptr(), ki.data_ptr(), kp.data_ptr(),
                               ptr(km), ptr(ks), vc.data_ptr(), vi.data_ptr(), vp.data_ptr(), ptr(vm), ptr(vs), b, hkv,
                               hq, tokens_arg, key.token_stride, kc.shape[1], vc.shape[1], 0, 500000.0, inv.data_ptr(),
                               128 ** -0.5, splits, qrf.data_ptr(), win_k.data_ptr(), win_v.data_ptr(), win_k.shape[2],
                               state.data_ptr(), ws.data_ptr(), ws.numel(), out.data_ptr(),
                               ext._stream(torch.device(DEV)))
    ext.check(rc, launches=2)
    torch.cuda.synchronize()
    assert int(ws[:4].view(torch.int32).item()) == 0, "kernel status word set"
    return out.reshape(b, hq, 1, 128)


@pytest.mark.parametrize("sparsity,bits,layout", PLANS)
def test_counts_from_the_step_state_match_the_by_value_call(sparsity, bits, layout):
    from reskv_b200 import ResKVKernelConfig, attention, compress
    from reskv_b200.synthetic import gaussian, mixture

    b, hkv, hq, t, live, cap = 2, 2, 8, 640, 20, 96
    k = mixture(b, hkv, t + cap, seed=31, device=DEV)
    v = mixture(b, hkv, t + cap, seed=32, device=DEV)
    cfg = ResKVKernelConfig(sparsity=sparsity, bits=bits, layout=layout, kmeans_iterations=3)
    cache = compress(k[:, :, :t].contiguous(), v[:, :, :t].contiguous(), cfg)
    cache.key, cache.value = cache.key.reserve(1024), cache.value.reserve(1024)
    pos = t + live - 1
    inv = 500000.0 ** (-torch.arange(64, device=DEV).float() / 64)
    q = gaussian(b, hq, 1, 128, seed=33, device=DEV)
    qr = _rope(q, pos, inv)
    win_k = torch.zeros((b, hkv, cap, 128), dtype=torch.float16, device=DEV)
    win_v = torch.zeros_like(win_k)
    for j in range(live):
        win_k[:, :, j] = _rope(k[:, :, t + j], t + j, inv)
    win_v[:, :, :live] = v[:, :, t:t + live]
    want = attention(q, cache, position=pos, recent=(qr, win_k[:, :, :live].contiguous(), win_v[:, :, :live].contiguous()))

    def state(tokens):
        return torch.tensor([pos, live, tokens, 0], dtype=torch.int32, device=DEV)

    # count by value (state says -1), count from the state with a stale (smaller) launch argument,
    # padded centroid tables, and a split count that leaves the last split without a tile
    got = _step(cache, q, qr, win_k, win_v, state(-1), t, 0)
    torch.testing.assert_close(got.float(), want.float(), atol=2e-3, rtol=1e-2)
    got = _step(cache, q, qr, win_k, win_v, state(t), 128, 0, rows=64)
    torch.testing.assert_close(got.float(), want.float(), atol=2e-3, rtol=1e-2)
    got = _step(cache, q, qr, win_k, win_v, state(t), 9 * 64, 4, rows=64)  # 10 tiles over 4 splits: 3,3,3,1
    torch.testing.assert_close(got.float(), want.float(), atol=2e-3, rtol=1e-2)
    got = _step(cache, q, qr, win_k, win_v, state(t - 64), t, 4)  # 9 tiles over 4 splits: the last split is empty
    short = compress(k[:, :, :t].contiguous(), v[:, :, :t].contiguous(), cfg)
    # the first t - 64 tokens of the same cache, by value
    from reskv_b200.tensors import CompressedTensor

    def head(x):
        return CompressedTensor._window(x.centroids, x._buffers, t - 64, x.plan)

    short.key, short.value = head(cache.key), head(cache.value)
    want_short = attention(q, short, position=pos, recent=(qr, win_k[:, :, :live].contiguous(), win_v[:, :, :live].contiguous()))
    torch.testing.assert_close(got.float(), want_short.float(), atol=2e-3, rtol=1e-2)


def test_window_append_and_advance():
    from reskv_b200 import _extension as ext

    lib = ext.library()
    b, hkv, cap = 2, 3, 8
    win = [torch.zeros((b * hkv, cap, 128), dtype=torch.float16, device=DEV) for _ in range(3)]
    new = [torch.randn((b * hkv, 128), device=DEV).half() for _ in range(3)]
    state = torch.tensor([100, 4, 7, 0], dtype=torch.int32, device=DEV)
    stream = ext._stream(torch.device(DEV))
    ext.check(lib.reskv_step_advance(state.data_ptr(), 0, 1, stream))
    ext.check(lib.reskv_window_append(*(w.data_ptr() for w in win), *(n.data_ptr() for n in new), b, hkv, cap,
                                      state.data_ptr(), stream))
    ext.check(lib.reskv_step_advance(state.data_ptr(), 1, 0, stream))
    torch.cuda.synchronize()
    assert state.tolist() == [101, 5, 7, 0]
    for w, n in zip(win, new):
        assert torch.equal(w[:, 4], n)
        assert not w[:, :4].any() and not w[:, 5:].any()

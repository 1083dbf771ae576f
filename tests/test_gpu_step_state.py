"""Decode driven by a device-side step state (the entry points a CUDA-graph decode
loop uses): results must equal the by-value ``attention()`` call for the same cache,
whether the compressed token count comes from the launch arguments or from the state."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
PLANS = [(0.75, 16, "unstructured"), (0.5, 16, "unstructured"), (0.5, 16, "tiled"), (0.75, 16, "structured"),
         (0.5, 4, "unstructured"), (0.5, 2, "unstructured"), (0.75, 4, "structured"), (0.5, 4, "compact")]


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


def _step(cache, q, qr, win_k, win_v, state, tokens_arg, splits, rows=None, expect_status=0):
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
    layout = {"unstructured": ext.LAYOUT_UNSTRUCTURED, "tiled": ext.LAYOUT_TILED, "structured": ext.LAYOUT_STRUCTURED,
              "compact": ext.LAYOUT_COMPACT}[plan.layout]
    need = lib.reskv_decode_bitmap_fp16_workspace_bytes(b, hkv, hq, 1 << 16, 64)
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    out = torch.empty((b * hq, 128), dtype=torch.float16, device=DEV)
    inv = (500000.0 ** (-torch.arange(64, device=DEV).float() / 64)).contiguous()

    def ptr(t):
        return None if t is None else t.data_ptr()

    qf, qrf = q.reshape(b * hq, 128).contiguous(), qr.reshape(b * hq, 128).contiguous()
    nnz = kp.shape[2] * 32 // plan.bits if plan.layout == "compact" else kp.shape[2]
    rc = lib.reskv_decode_step(layout, plan.bits, nnz, qf.data_ptr(), kc.data_ptr(), ki.data_ptr(), kp.data_ptr(),
                               ptr(km), ptr(ks), vc.data_ptr(), vi.data_ptr(), vp.data_ptr(), ptr(vm), ptr(vs), b, hkv,
                               hq, tokens_arg, key.token_stride, kc.shape[1], vc.shape[1], 0, 500000.0, inv.data_ptr(),
                               128 ** -0.5, splits, qrf.data_ptr(), win_k.data_ptr(), win_v.data_ptr(), win_k.shape[2],
                               state.data_ptr(), ws.data_ptr(), ws.numel(), out.data_ptr(),
                               ext._stream(torch.device(DEV)))
    ext.check(rc, launches=2)
    torch.cuda.synchronize()
    assert int(ws[:4].view(torch.int32).item()) == expect_status, "unexpected kernel status word"
    return out.reshape(b, hq, 1, 128)


@pytest.mark.parametrize("sparsity,bits,layout", PLANS)
def test_counts_from_the_step_state_match_the_by_value_call(sparsity, bits, layout, kernel_variant):
    from reskv_b200 import ResKVKernelConfig, attention, compress

    if layout == "compact" and kernel_variant == "simt":
        pytest.skip("the compact layout has no warp-per-token kernel")
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
    if sparsity == 0.75 and bits == 16 and layout == "unstructured":
        # counts beyond the buffers are cut (window tokens to the capacity, compressed tokens to the token
        # stride) and reported: bit RESKV_STATUS_STATE_RANGE (2) of the status word, no fault
        over = torch.tensor([pos, cap + 1, t, 0], dtype=torch.int32, device=DEV)
        _step(cache, q, qr, win_k, win_v, over, t, 0, expect_status=2)
        if kernel_variant == "tensor-core":
            over = torch.tensor([pos + 4096, live, cache.key.token_stride + 1, 0], dtype=torch.int32, device=DEV)
            _step(cache, q, qr, win_k, win_v, over, t, 0, expect_status=2)
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


def test_layer_helpers_match_tensor_ops():
    """RMS norm, QKV split + RoPE + window append, SiLU * up against plain tensor arithmetic."""
    from reskv_b200 import _extension as ext
    from reskv_b200.models.llama import _rms_norm, _rope

    lib = ext.library()
    stream = ext._stream(torch.device(DEV))
    g = torch.Generator(device=DEV).manual_seed(5)
    b, hq, hkv, d, ffn, cap, pos, live = 3, 8, 2, 512, 640, 12, 777, 5

    x = (torch.randn(b, d, generator=g, device=DEV) * 3).half()
    w = torch.randn(d, generator=g, device=DEV).half()
    out = torch.empty_like(x)
    ext.check(lib.reskv_rms_norm(x.data_ptr(), w.data_ptr(), out.data_ptr(), b, d, 1e-5, stream))
    torch.testing.assert_close(out, _rms_norm(x, w, 1e-5), atol=2e-3, rtol=2e-3)

    qkv = torch.randn(b, (hq + 2 * hkv) * 128, generator=g, device=DEV).half()
    inv = (500000.0 ** (-torch.arange(64, device=DEV).float() / 64)).contiguous()
    state = torch.tensor([pos, live, -1, 0], dtype=torch.int32, device=DEV)
    q_raw, q_rot = (torch.empty(b * hq, 128, dtype=torch.float16, device=DEV) for _ in range(2))
    k_rot, v_out = (torch.empty(b * hkv, 128, dtype=torch.float16, device=DEV) for _ in range(2))
    win = [torch.zeros(b * hkv, cap, 128, dtype=torch.float16, device=DEV) for _ in range(3)]
    ext.check(lib.reskv_rope_split(qkv.data_ptr(), b, hq, hkv, inv.data_ptr(), state.data_ptr(), q_raw.data_ptr(),
                                   q_rot.data_ptr(), k_rot.data_ptr(), v_out.data_ptr(), *(t.data_ptr() for t in win),
                                   cap, stream))
    torch.cuda.synchronize()
    q, k, v = qkv.split((hq * 128, hkv * 128, hkv * 128), dim=-1)
    ang = float(pos) * inv
    cos, sin = ang.cos()[None], ang.sin()[None]
    want_q = _rope(q.reshape(b, hq, 1, 128), cos, sin).reshape(b * hq, 128)
    want_k = _rope(k.reshape(b, hkv, 1, 128), cos, sin).reshape(b * hkv, 128)
    assert torch.equal(q_raw, q.reshape(b * hq, 128)) and torch.equal(v_out, v.reshape(b * hkv, 128))
    torch.testing.assert_close(q_rot, want_q, atol=2e-3, rtol=2e-3)
    torch.testing.assert_close(k_rot, want_k, atol=2e-3, rtol=2e-3)
    assert torch.equal(win[0][:, live - 1], k_rot) and torch.equal(win[1][:, live - 1], k.reshape(b * hkv, 128))
    assert torch.equal(win[2][:, live - 1], v_out)
    for t in win:
        assert not t[:, :live - 1].any() and not t[:, live:].any()

    gu = torch.randn(b, 2 * ffn, generator=g, device=DEV).half()
    act = torch.empty(b, ffn, dtype=torch.float16, device=DEV)
    ext.check(lib.reskv_silu_mul(gu.data_ptr(), act.data_ptr(), b, ffn, stream))
    want = torch.nn.functional.silu(gu[:, :ffn]) * gu[:, ffn:]
    torch.testing.assert_close(act, want, atol=1e-3, rtol=2e-3)

"""Loader and operator tables of the native library.

The reference JIT-builds one pybind11 module per kernel family and plan
(reskv/_extension.py:14-61) and calls its functions positionally
(reskv/compression.py:90-99, reskv/_attention.py:59-143).  Here one
ahead-of-time ``libreskv_b200.so`` (sm_100a, C ABI, see
``include/reskv_b200.h``) is opened with ``ctypes``; ``load_extension`` keeps the
reference's signature and returns an object that exposes the same operator
names with the same positional arguments and return values.  Tensors stay
torch-owned: outputs and scratch memory are allocated here with ``torch.empty``
and the kernels run on the current CUDA stream.

There is no CPU or eager fallback: a missing library, a device that is not
compute capability 10.x, or a failing kernel call raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p
from functools import lru_cache
from pathlib import Path

import torch

from .config import KernelPlan

_LIB_PATH = Path(__file__).resolve().parent / "csrc" / "libreskv_b200.so"
_FAMILIES = ("compression", "attention", "cluster_mass")

ERR_INVALID, ERR_WORKSPACE, ERR_CUDA, ERR_LIMIT = -1, -2, -3, -4

# name -> (restype, argtypes): exactly the declarations of include/reskv_b200.h
_P, _I, _L, _F, _Z = c_void_p, c_int, c_int64, c_float, c_size_t
SIGNATURES = {
    "reskv_last_error": (c_char_p, []),
    "reskv_version": (_I, []),
    "reskv_decode_bitmap_fp16_workspace_bytes": (_Z, [_I, _I, _I, _I, _I]),
    "reskv_decode_bitmap_fp16": (
        _I,
        [_P] * 9 + [_I, _I, _I, _I, _L, _I, _I, _I, _I, _I, _F, _P, _F, _I, _P, _P, _P, _I, _P, _Z, _P, _P, _P, _P],
    ),
    "reskv_decode_packed": (
        _I,
        [_I, _I] + [_P] * 11 + [_I, _I, _I, _I, _L, _I, _I, _I, _I, _F, _P, _F, _I, _P, _P, _P, _I, _P, _Z, _P, _P, _P, _P],
    ),
    "reskv_decode_bitmap_fp16_noalloc": (
        _I,
        [_P] * 9 + [_I, _I, _I, _I, _L, _I, _I, _I, _I, _I, _F, _P, _F, _I, _P, _P, _P, _I, _P, _P, _P, _P],
    ),
    "reskv_encode_compact": (_I, [_P, _P, _P, _I, _I, _I, _L, _I, _I, _I, _P, _P, _P, _L, _P]),
    "reskv_decode_compact": (
        _I,
        [_I, _I] + [_P] * 11 + [_I, _I, _I, _I, _L, _I, _I, _I, _I, _F, _P, _F, _I, _P, _P, _P, _I, _P, _Z, _P, _P, _P, _P],
    ),
    "reskv_window_append": (_I, [_P] * 6 + [_I, _I, _I, _P, _P]),
    "reskv_window_write": (_I, [_P] * 6 + [_I, _I, _I, _I, _P]),
    "reskv_decode_step": (
        _I,
        [_I, _I, _I] + [_P] * 11 + [_I, _I, _I, _I, _L, _I, _I, _I, _F, _P, _F, _I, _P, _P, _P, _I, _P, _P, _Z, _P, _P],
    ),
    "reskv_step_advance": (_I, [_P, _I, _I, _P]),
    "reskv_rms_norm": (_I, [_P, _P, _P, _I, _I, _F, _P]),
    "reskv_rope_split": (_I, [_P, _I, _I, _I, _P, _P] + [_P] * 7 + [_I, _P]),
    "reskv_silu_mul": (_I, [_P, _P, _I, _I, _P]),
    "reskv_decode_auto_splits": (_I, [_I, _I, _I]),
    "reskv_decode_noalloc_status": (_I, [_P, _P]),
    "reskv_decode_set_variant": (_I, [_I]),
    "reskv_decode_set_timing_events": (_I, [_P, _P]),
    "reskv_merge_recent_scores": (_I, [_P] * 5 + [_I, _I, _I, _I, _P, _P]),
    "reskv_merge_recent_qk": (_I, [_P] * 6 + [_I, _I, _I, _I, _F, _P, _P]),
    "reskv_encode_bitmap_fp16": (_I, [_P, _P, _P, _I, _I, _I, _L, _I, _I, _P, _P, _L, _P]),
    "reskv_encode_quantized": (_I, [_P, _P, _P, _I, _I, _I, _L, _I, _I, _I, _P, _P, _L, _P]),
    "reskv_encode_tiled_fp16": (_I, [_P, _P, _P, _I, _I, _I, _L, _I, _I, _I, _P, _P, _L, _P]),
    "reskv_encode_structured_int4": (_I, [_P, _P, _P, _I, _I, _I, _L, _I, _P, _P, _P, _L, _P]),
    "reskv_compress_group": (
        _I,
        [_I, _I, _I, _P, _P, _I, _I, _I, _L] + [_P, _I, _P, _I, _P, _P, _P, _P, _L] * 2 + [_I, _P, _P],
    ),
    "reskv_window_shift": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "reskv_kmeans_workspace_bytes": (_Z, [_I, _I, _I]),
    "reskv_kmeans": (_I, [_P, _I, _I, _I, _L, _I, _I, _I, _P, _Z, _P, _P, _P]),
    "reskv_kmeans_status": (_I, [_P, _I, _I, _I, _P, _P]),
    "reskv_kmeans_incremental": (_I, [_P, _I, _I, _I, _L, _P, _I, _P, _I, _P, _P]),
}


@lru_cache(maxsize=1)
def library() -> ctypes.CDLL:
    """The native library, with argument types set.  Raises if it was not built."""
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python -m reskv_b200.csrc.build` "
            "(needs nvcc; there is no fallback path)"
        )
    lib = ctypes.CDLL(str(_LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = restype, argtypes
    return lib


# Kernels launched through this module since import (bench.py reports it).
launch_count = 0


def check(rc: int, launches: int = 1) -> None:
    """Count the launches of a successful call; turn a negative return code into
    the exception the reference would raise: argument problems are ``ValueError`` (the reference's TORCH_CHECKs surface as
    RuntimeError subclasses, its Python checks as ValueError; callers match on
    the message), everything else ``RuntimeError``."""
    if rc >= 0:
        global launch_count
        launch_count += launches
        return
    msg = library().reskv_last_error().decode()
    if rc in (ERR_INVALID, ERR_LIMIT):
        raise ValueError(msg)
    raise RuntimeError(msg)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_CHECK_STATUS = os.environ.get("RESKV_CHECK_STATUS") == "1"


def device_index_of(device) -> int:
    """Ordinal of a CUDA device; an index-less ``cuda`` device means the current one."""
    index = torch.device(device).index if not isinstance(device, int) else device
    return torch.cuda.current_device() if index is None else int(index)


class BoundLibrary:
    """The native library with one CUDA device made current around every call.

    The C entry points launch on the current device and cache per-device facts
    (SM count, kernel attributes, built-in scratch) against it, like the reference's
    ops do under ``CUDAGuard(tensor.device())`` (cluster_mass.cu:1187, attention.cu:684,
    compression.cu:396).  Tensors of ``cuda:1`` used while ``cuda:0`` is current would
    otherwise be handed to a launch on the wrong GPU.
    """

    def __init__(self, lib: ctypes.CDLL, device_index: int):
        self._lib, self._index = lib, int(device_index)

    def __getattr__(self, name):
        fn, index = getattr(self._lib, name), self._index

        def call(*args):
            if torch.cuda.current_device() == index:
                return fn(*args)
            with torch.cuda.device(index):
                return fn(*args)

        self.__dict__[name] = call
        return call


def bound_library(device) -> BoundLibrary:
    """``library()`` bound to ``device`` (a ``torch.device``, tensor device or ordinal)."""
    return BoundLibrary(library(), device_index_of(device))


def _same_device(device_index: int, *tensors) -> None:
    for t in tensors:
        if t is not None and (not t.is_cuda or device_index_of(t.device) != device_index):
            raise ValueError(f"all tensors of this call must live on cuda:{device_index}, got one on {t.device}")


class _Ops:
    """Base of the operator tables: remembers the plan and device of the load."""

    def __init__(self, plan: KernelPlan | None, device_index: int):
        self.plan = plan
        self.device = torch.device("cuda", device_index)
        self.lib = BoundLibrary(library(), device_index)


class CompressionOps(_Ops):
    """``compression`` family (reference pybind module compression.cu:508-512)."""

    def _dims(self, x, centroids, ids):
        if x.dtype != torch.float16 or centroids.dtype != torch.float16 or ids.dtype != torch.int32:
            raise ValueError("compression ops expect FP16 x/centroids and int32 ids")
        if x.ndim != 4 or centroids.ndim != 4 or ids.ndim != 3 or x.shape[3] != 128 or centroids.shape[3] != 128:
            raise ValueError("compression ops expect x[B,H,T,128], centroids[B,H,C,128], ids[B,H,T]")
        stride = token_stride_of(x)
        if stride is None or not (centroids.is_contiguous() and ids.is_contiguous()):
            raise ValueError("compression ops expect contiguous tensors (x may be a token slice of a dense buffer)")
        _same_device(self.device.index, x, centroids, ids)
        b, h, t, _ = x.shape
        return b, h, t, centroids.shape[2], stride

    def compress_bitmap_fp16(self, x, centroids, ids, nnz):
        """Unstructured FP16 -> (payload f16 [B,H,T,nnz], bitmap i64 [B,H,T,2]).
        The reference has no native op for this layout (torch ops,
        compression.py:75-89); it is one kernel here."""
        b, h, t, c, xs = self._dims(x, centroids, ids)
        payload = torch.empty((b, h, t, nnz), dtype=torch.float16, device=x.device)
        bitmap = torch.empty((b, h, t, 2), dtype=torch.int64, device=x.device)
        check(self.lib.reskv_encode_bitmap_fp16(x.data_ptr(), centroids.data_ptr(), ids.data_ptr(), b, h, t, xs, c,
                                                nnz, payload.data_ptr(), bitmap.data_ptr(), t, _stream(x.device)))
        return payload, bitmap

    def compress_fp16(self, x, centroids, ids, nnz, structured):
        b, h, t, c, xs = self._dims(x, centroids, ids)
        values = torch.empty((b, h, t, nnz), dtype=torch.float16, device=x.device)
        meta = torch.empty((b, h, t, 4), dtype=torch.int32, device=x.device)
        check(self.lib.reskv_encode_tiled_fp16(x.data_ptr(), centroids.data_ptr(), ids.data_ptr(), b, h, t, xs, c, nnz,
                                               int(bool(structured)), values.data_ptr(), meta.data_ptr(), t,
                                               _stream(x.device)))
        return values, meta

    def compress_quantized(self, x, centroids, ids, nnz, bits):
        b, h, t, c, xs = self._dims(x, centroids, ids)
        words = torch.empty((b, h, t, 4 * bits), dtype=torch.int32, device=x.device)
        scale = torch.empty((b, h, t), dtype=torch.float16, device=x.device)
        check(self.lib.reskv_encode_quantized(x.data_ptr(), centroids.data_ptr(), ids.data_ptr(), b, h, t, xs, c, nnz,
                                              bits, words.data_ptr(), scale.data_ptr(), t, _stream(x.device)))
        return words, scale

    def compress_compact(self, x, centroids, ids, nnz, bits):
        """Compact quantised layout (not in the reference): ``(words i32 [B,H,T,nnz*bits/32],
        bitmap i64 [B,H,T,2], scale f16 [B,H,T])``."""
        b, h, t, c, xs = self._dims(x, centroids, ids)
        words = torch.empty((b, h, t, nnz * bits // 32), dtype=torch.int32, device=x.device)
        bitmap = torch.empty((b, h, t, 2), dtype=torch.int64, device=x.device)
        scale = torch.empty((b, h, t), dtype=torch.float16, device=x.device)
        check(self.lib.reskv_encode_compact(x.data_ptr(), centroids.data_ptr(), ids.data_ptr(), b, h, t, xs, c, nnz, bits,
                                            words.data_ptr(), bitmap.data_ptr(), scale.data_ptr(), t, _stream(x.device)))
        return words, bitmap, scale

    def compress_structured_int4(self, x, centroids, ids):
        b, h, t, c, xs = self._dims(x, centroids, ids)
        packed = torch.empty((b, h, t, 4), dtype=torch.int32, device=x.device)
        meta = torch.empty((b, h, t, 2), dtype=torch.int32, device=x.device)
        scale = torch.empty((b, h, t), dtype=torch.float16, device=x.device)
        check(self.lib.reskv_encode_structured_int4(x.data_ptr(), centroids.data_ptr(), ids.data_ptr(), b, h, t, xs, c,
                                                    packed.data_ptr(), meta.data_ptr(), scale.data_ptr(), t,
                                                    _stream(x.device)))
        return packed, meta, scale

    def kmeans(self, x, count, iterations, value, exact=False, warp_mma=False, return_status=False):
        """Lloyd clustering -> (centroids f16 [B,H,C,128], ids i32 [B,H,T]).  ``exact``: accumulate the cluster
        sums as integers (correctly rounded means) instead of FP32 partial sums on the tensor cores; ``warp_mma``:
        the mma.sync form of the tensor-core sums instead of the tcgen05 one; ``return_status``: also return the
        kernels' status word (synchronises the stream)."""
        if x.dtype != torch.float16 or x.ndim != 4 or x.shape[3] != 128 or token_stride_of(x) is None:
            raise ValueError("kmeans expects FP16 x[B,H,T,128], dense or a token slice of a dense buffer")
        _same_device(self.device.index, x)
        b, h, t, _ = x.shape
        xs = token_stride_of(x)
        need = self.lib.reskv_kmeans_workspace_bytes(b, h, count)
        if need == 0:
            raise ValueError("kmeans: cluster count must be in [1,64]")
        ws = torch.empty(need, dtype=torch.uint8, device=x.device)
        centroids = torch.empty((b, h, count, 128), dtype=torch.float16, device=x.device)
        ids = torch.empty((b, h, t), dtype=torch.int32, device=x.device)
        flags = int(bool(value)) | (2 if exact else 0) | (4 if warp_mma else 0)
        check(self.lib.reskv_kmeans(x.data_ptr(), b, h, t, xs, count, iterations, flags, ws.data_ptr(), need,
                                    centroids.data_ptr(), ids.data_ptr(), _stream(x.device)), launches=1 + 2 * iterations)
        if return_status:
            word = ctypes.c_uint32(0xFFFFFFFF)
            check(self.lib.reskv_kmeans_status(ws.data_ptr(), b, h, count, ctypes.addressof(word), _stream(x.device)))
            return centroids, ids, word.value
        return centroids, ids

    def kmeans_incremental(self, x, centroids, append):
        """Decode-time step -> (centroids f16 [B,H,C or C+1,128], ids i32 [B,H,T])."""
        _same_device(self.device.index, x, centroids)
        b, h, t, _ = x.shape
        xs = token_stride_of(x)
        if x.dtype != torch.float16 or xs is None:
            raise ValueError("kmeans_incremental expects FP16 x[B,H,T,128], dense or a token slice of a dense buffer")
        old = centroids.shape[2]
        new = old + int(bool(append))
        centroids = centroids.contiguous()
        out = torch.empty((b, h, new, 128), dtype=torch.float16, device=x.device)
        ids = torch.empty((b, h, t), dtype=torch.int32, device=x.device)
        check(self.lib.reskv_kmeans_incremental(x.data_ptr(), b, h, t, xs, centroids.data_ptr(), old, out.data_ptr(),
                                                new, ids.data_ptr(), _stream(x.device)))
        return out, ids


    def compress_group(self, plan: KernelPlan, x_k, x_v, sides, seq_len: int):
        """One decode group of K and V clustered, packed and written behind token ``seq_len`` of the capacity
        buffers, in one library call.  ``sides`` = for K then V ``(old table f16 [B*H,C,128], new table f16
        [B,H,C or C+1,128] (the old one when the count stays), buffers (ids i8, payload, metadata, scale)
        [B,H,capacity,...])``.  ``x_k`` / ``x_v`` share one token stride."""
        b, h, t, _ = x_k.shape
        xs = token_stride_of(x_k)
        if x_k.dtype != torch.float16 or x_v.dtype != torch.float16 or xs is None or xs != token_stride_of(x_v):
            raise ValueError("compress_group expects FP16 x[B,H,T,128] of one token stride")
        layout = {"unstructured": LAYOUT_UNSTRUCTURED, "tiled": LAYOUT_TILED, "structured": LAYOUT_STRUCTURED,
                  "compact": LAYOUT_COMPACT}[plan.layout]
        args = []
        for old, new, buffers in sides:
            _same_device(self.device.index, old, new, *buffers)
            ids = buffers[0]
            if ids.dtype != torch.int8 or not all(buf is None or buf.is_contiguous() for buf in buffers):
                raise ValueError("compress_group expects contiguous capacity buffers with int8 ids")
            args += [old.data_ptr(), old.shape[1], new.data_ptr(), new.shape[2]]
            args += [0 if buf is None else buf.data_ptr() for buf in buffers] + [ids.shape[2]]
        scratch = torch.empty((2, b * h, t), dtype=torch.int32, device=x_k.device)
        check(self.lib.reskv_compress_group(layout, plan.bits, plan.nnz, x_k.data_ptr(), x_v.data_ptr(), b, h, t, xs, *args,
                                            seq_len, scratch.data_ptr(), _stream(x_k.device)), launches=5)


def token_stride_of(x: torch.Tensor):
    """Tokens between consecutive (sequence, head) units of ``x[B,H,T,128]`` when ``x`` is dense or a token slice of
    a dense ``[B,H,capacity,128]`` buffer (rows of 128 contiguous, units evenly spaced), else ``None``.  The kernels
    take that stride next to the token count, so such a slice needs no copy."""
    b, h, t, d = x.shape
    if d != 128 or x.stride(3) != 1 or (t > 1 and x.stride(2) != 128):
        return None
    if h > 1:
        step = x.stride(1)
    elif b > 1:
        step = x.stride(0)
    else:
        return t
    if step % 128 or step // 128 < t or (h > 1 and b > 1 and x.stride(0) != h * step):
        return None
    return step // 128


def _token_stride(rows: torch.Tensor, width: int) -> int:
    """Tokens between units of a ``[units, T, width]`` (or ``[units, T]``) view."""
    if rows.shape[0] == 1:
        return rows.shape[1]
    return rows.stride(0) // width


LAYOUT_UNSTRUCTURED, LAYOUT_TILED, LAYOUT_STRUCTURED, LAYOUT_COMPACT = 0, 1, 2, 3


def _decode(lib, layout, bits, q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, kh, nh, start_pos, pos_q, rope_theta, scale,
            splits, inv_freq, return_stats=True, recent=None):
    """Allocate outputs and scratch, call the decode entry point of a layout.

    ``layout is None`` selects the unstructured FP16 bitmap kernel, ``LAYOUT_COMPACT``
    ``reskv_decode_compact``, anything else ``reskv_decode_packed``.  ``recent = (q_rot [B*nh,128], k_rot, v [B,kh,Tr,128])``
    folds a dense window into the same launch pair.
    """
    _same_device(lib._index, q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, inv_freq, *(recent or ()))
    bnh = q.shape[0]
    b = bnh // nh
    t, width = kp.shape[1], kp.shape[2]
    stride = _token_stride(kp, width)
    for rows in (ki, km, ks, vi, vp, vm, vs):
        if rows is not None and rows.numel() and _token_stride(rows, rows.shape[2] if rows.ndim == 3 else 1) != stride:
            raise ValueError("K and V cache tensors must share one token stride")
    dev = q.device
    need = lib.reskv_decode_bitmap_fp16_workspace_bytes(b, kh, nh, t, int(splits))
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
    if _CHECK_STATUS:
        ws[:256].zero_()
    out = torch.empty((bnh, 128), dtype=torch.float16, device=dev)
    m = torch.empty(bnh, dtype=torch.float32, device=dev) if return_stats else None
    l = torch.empty(bnh, dtype=torch.float32, device=dev) if return_stats else None
    rq = rk = rv = None
    tr = 0
    if recent is not None and recent[1].shape[2] > 0:
        rq, rk, rv = (x.contiguous() for x in recent)
        tr = rk.shape[2]
    tail = (b, kh, nh, t, stride, kc.shape[1], vc.shape[1])
    rest = (int(start_pos), int(pos_q), float(rope_theta), _ptr(inv_freq), float(scale), int(splits), _ptr(rq),
            _ptr(rk), _ptr(rv), tr, ws.data_ptr(), ws.numel(), out.data_ptr(), _ptr(m), _ptr(l), _stream(dev))
    if layout is None:
        rc = lib.reskv_decode_bitmap_fp16(q.data_ptr(), kc.data_ptr(), ki.data_ptr(), kp.data_ptr(), km.data_ptr(),
                                          vc.data_ptr(), vi.data_ptr(), vp.data_ptr(), vm.data_ptr(), *tail, width,
                                          *rest)
    elif layout == LAYOUT_COMPACT:
        rc = lib.reskv_decode_compact(bits, width * 32 // bits, q.data_ptr(), kc.data_ptr(), ki.data_ptr(), kp.data_ptr(),
                                      _ptr(km), _ptr(ks), vc.data_ptr(), vi.data_ptr(), vp.data_ptr(), _ptr(vm),
                                      _ptr(vs), *tail, *rest)
    else:
        rc = lib.reskv_decode_packed(layout, bits, q.data_ptr(), kc.data_ptr(), ki.data_ptr(), kp.data_ptr(),
                                     _ptr(km), _ptr(ks), vc.data_ptr(), vi.data_ptr(), vp.data_ptr(), _ptr(vm),
                                     _ptr(vs), *tail, *rest)
    check(rc, launches=2)
    if _CHECK_STATUS:
        status = int(ws[:4].view(torch.int32).item())
        if status:
            raise RuntimeError(f"decode: device status {status:#x} (bounded wait ran out)")
    return (out, m, l) if return_stats else (out,)


class ClusterMassOps(_Ops):
    """``cluster_mass`` family (reference pybind module cluster_mass.cu:1511-1516)."""

    def decode_fp16(self, q, kc, ki, kp, km, vc, vi, vp, vm, kh, nh, start_pos, pos_q, rope_theta, scale,
                    return_stats=True, splits=0, inv_freq=None, recent=None):
        """Unstructured FP16 bitmap decode -> ``(out, m, l)`` (``(out,)`` without
        stats), as cluster_mass.cu:1177-1296.  ``recent`` (not part of the
        reference signature) fuses the dense window into the same call."""
        return _decode(self.lib, None, 16, q, kc, ki, kp, km, None, vc, vi, vp, vm, None, kh, nh, start_pos, pos_q,
                       rope_theta, scale, splits, inv_freq, return_stats, recent)

    def decode_structured_fp16(self, q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, kh, nh, start_pos, pos_q, rope_theta,
                               scale, return_stats=True, splits=0, inv_freq=None, recent=None):
        return _decode(self.lib, LAYOUT_STRUCTURED, 16, q, kc, ki, kp, km, None, vc, vi, vp, vm, None, kh, nh,
                       start_pos, pos_q, rope_theta, scale, splits, inv_freq, return_stats, recent)

    def decode_structured_int4(self, q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, kh, nh, start_pos, pos_q, rope_theta,
                               scale, return_stats=True, splits=0, inv_freq=None, recent=None):
        return _decode(self.lib, LAYOUT_STRUCTURED, 4, q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, kh, nh, start_pos,
                       pos_q, rope_theta, scale, splits, inv_freq, return_stats, recent)

    def merge_recent(self, out, m, l, scores, v_recent, kh, nh):
        _same_device(self.device.index, out, m, l, scores, v_recent)
        b = out.shape[0] // nh
        merged = torch.empty_like(out)
        check(self.lib.reskv_merge_recent_scores(out.data_ptr(), m.data_ptr(), l.data_ptr(), scores.data_ptr(),
                                                 v_recent.data_ptr(), b, kh, nh, v_recent.shape[2], merged.data_ptr(),
                                                 _stream(out.device)))
        return merged


class AttentionOps(_Ops):
    """``attention`` family (reference pybind module attention.cu:1350-1355)."""

    def decode_fp16(self, q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, kh, nh, start_pos, pos_q, rope_theta, scale,
                    splits=0, inv_freq=None, recent=None):
        """Tiled (64 values per token) or 4:16 structured (32 values) FP16 decode."""
        layout = LAYOUT_TILED if kp.shape[2] == 64 else LAYOUT_STRUCTURED
        return _decode(self.lib, layout, 16, q, kc, ki, kp, km, None, vc, vi, vp, vm, None, kh, nh, start_pos, pos_q,
                       rope_theta, scale, splits, inv_freq, True, recent)

    def decode_int4(self, q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, kh, nh, start_pos, pos_q, rope_theta, scale,
                    splits=0, inv_freq=None, recent=None):
        return _decode(self.lib, LAYOUT_STRUCTURED, 4, q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, kh, nh, start_pos,
                       pos_q, rope_theta, scale, splits, inv_freq, True, recent)

    def decode_quantized(self, q, kc, ki, kp, ks, vc, vi, vp, vs, kh, nh, start_pos, pos_q, rope_theta, scale, k_bits,
                         v_bits, splits=0, inv_freq=None, recent=None):
        if k_bits != v_bits or k_bits not in (2, 4):
            raise ValueError("decode_quantized expects equal key and value bit widths of 2 or 4")
        return _decode(self.lib, LAYOUT_UNSTRUCTURED, k_bits, q, kc, ki, kp, None, ks, vc, vi, vp, None, vs, kh, nh,
                       start_pos, pos_q, rope_theta, scale, splits, inv_freq, True, recent)

    def decode_compact(self, q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, kh, nh, start_pos, pos_q, rope_theta, scale,
                       bits, splits=0, inv_freq=None, recent=None):
        """Compact quantised layout (not in the reference): bitmap + codes of the retained coordinates."""
        return _decode(self.lib, LAYOUT_COMPACT, bits, q, kc, ki, kp, km, ks, vc, vi, vp, vm, vs, kh, nh, start_pos,
                       pos_q, rope_theta, scale, splits, inv_freq, True, recent)

    def merge_recent(self, out, m, l, q_rope, k_recent, v_recent, kh, nh, scale):
        _same_device(self.device.index, out, m, l, q_rope, k_recent, v_recent)
        b = out.shape[0] // nh
        merged = torch.empty_like(out)
        check(self.lib.reskv_merge_recent_qk(out.data_ptr(), m.data_ptr(), l.data_ptr(), q_rope.data_ptr(),
                                             k_recent.data_ptr(), v_recent.data_ptr(), b, kh, nh, k_recent.shape[2],
                                             float(scale), merged.data_ptr(), _stream(out.device)))
        return merged


_TABLES = {"compression": CompressionOps, "attention": AttentionOps, "cluster_mass": ClusterMassOps}


def load_extension(family: str, plan: KernelPlan | None = None, device_index: int | None = 0):
    """Operator table of one kernel family (reference _extension.py:14-61); ``device_index=None``
    means the current CUDA device.  See ``_load_extension`` for what is (not) built."""
    if device_index is None and family in _FAMILIES and torch.cuda.is_available():
        device_index = torch.cuda.current_device()
    return _load_extension(family, plan, device_index)


@lru_cache(maxsize=32)
def _load_extension(family: str, plan: KernelPlan | None = None, device_index: int | None = 0):
    """Operator table of one kernel family (reference _extension.py:14-61).

    Unlike the reference nothing is compiled here: the plan only selects
    template instances inside the prebuilt library at call time."""
    if family not in _FAMILIES:
        raise ValueError(f"unknown native family: {family}")
    if not torch.cuda.is_available():
        raise RuntimeError("ResKV B200 kernels need a CUDA device (there is no CPU path)")
    capability = torch.cuda.get_device_capability(device_index)
    if capability[0] != 10:
        raise RuntimeError(
            f"libreskv_b200 is built for sm_100a only; device {device_index} has compute capability "
            f"{capability[0]}.{capability[1]}"
        )
    return _TABLES[family](plan, device_index or 0)

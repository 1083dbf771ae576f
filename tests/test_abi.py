"""The C-ABI library: it loads, exports every declared symbol, and the Python
binding table matches the header (no compute calls: this runs without a GPU)."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "reskv_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    out = {}
    for m in re.finditer(r"([\w\s\*]+?)\b(reskv_\w+)\s*\(([^)]*)\)\s*;", text):
        args = [a.strip() for a in m.group(3).split(",") if a.strip() and a.strip() != "void"]
        out[m.group(2)] = (m.group(1).strip(), args)
    return out


@pytest.fixture(scope="module")
def lib():
    from reskv_b200.csrc.build import build

    return ctypes.CDLL(str(build()))


def test_every_declared_symbol_is_exported(lib):
    decl = declared_functions()
    assert len(decl) >= 14
    for name in decl:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def _ctype_of(c_arg: str):
    c_arg = c_arg.strip()
    if "*" in c_arg:
        return ctypes.c_char_p if c_arg.startswith("const char") else ctypes.c_void_p
    base = c_arg.split()[0] if " " in c_arg else c_arg
    return {"int": ctypes.c_int, "int64_t": ctypes.c_int64, "float": ctypes.c_float, "size_t": ctypes.c_size_t}[base]


def test_binding_table_matches_header():
    from reskv_b200._extension import SIGNATURES

    decl = declared_functions()
    assert set(SIGNATURES) == set(decl)
    for name, (ret, args) in decl.items():
        restype, argtypes = SIGNATURES[name]
        assert restype is _ctype_of(ret + (" x" if "*" not in ret else "")), name
        assert [_ctype_of(a) for a in args] == list(argtypes), name


def test_errors_are_reported_without_a_device(lib):
    lib.reskv_last_error.restype = ctypes.c_char_p
    lib.reskv_decode_auto_splits.argtypes = [ctypes.c_int] * 3
    assert lib.reskv_decode_auto_splits(0, 8, 100) == -1
    assert b"positive" in lib.reskv_last_error()
    lib.reskv_decode_bitmap_fp16_workspace_bytes.restype = ctypes.c_size_t
    lib.reskv_decode_bitmap_fp16_workspace_bytes.argtypes = [ctypes.c_int] * 5
    assert lib.reskv_decode_bitmap_fp16_workspace_bytes(1, 8, 32, 8128, 4) == 256 + 32 * 4 * (2 + 128 + 64) * 4
    lib.reskv_kmeans_workspace_bytes.restype = ctypes.c_size_t
    lib.reskv_kmeans_workspace_bytes.argtypes = [ctypes.c_int] * 3
    assert lib.reskv_kmeans_workspace_bytes(1, 8, 65) == 0
    assert lib.reskv_version() >= 100


def test_package_import_is_light():
    import subprocess
    import sys

    subprocess.run(
        [sys.executable, "-c",
         "import sys; import reskv_b200; assert 'torch' not in sys.modules; "
         "assert reskv_b200.ResKVKernelConfig().bits == 16; assert reskv_b200.ResKVConfig().bits == 16; "
         "assert 'torch' not in sys.modules"],
        check=True, cwd=ROOT)


def test_pointers_that_are_not_memory_of_the_current_device_are_refused():
    """Every entry point launches on the current device: host memory (here) or another GPU's memory is
    turned down with RESKV_ERR_INVALID before anything is launched."""
    import numpy as np

    from reskv_b200._extension import ERR_INVALID, library

    lib = library()
    t, nnz = 64, 32
    host = {name: np.zeros(shape, dtype) for name, shape, dtype in (
        ("q", (4, 128), np.float16), ("cen", (1, 32, 128), np.float16), ("ids", (1, t), np.int8),
        ("pay", (1, t, nnz), np.float16), ("bm", (1, t, 2), np.int64), ("ws", (1 << 20,), np.uint8),
        ("out", (4, 128), np.float16))}
    ptr = {k: v.ctypes.data for k, v in host.items()}
    assert all(p % 16 == 0 for p in ptr.values())
    rc = lib.reskv_decode_bitmap_fp16(ptr["q"], ptr["cen"], ptr["ids"], ptr["pay"], ptr["bm"], ptr["cen"], ptr["ids"],
                                      ptr["pay"], ptr["bm"], 1, 1, 4, t, t, 32, 32, nnz, 0, t, 500000.0, None, 0.088, 0,
                                      None, None, None, 0, ptr["ws"], host["ws"].size, ptr["out"], None, None, None)
    assert rc == ERR_INVALID
    assert b"decode_bitmap_fp16: q" in lib.reskv_last_error()
    x = np.zeros((1, 1, t, 128), np.float16)
    ids = np.zeros((1, 1, t), np.int32)
    rc = lib.reskv_encode_bitmap_fp16(x.ctypes.data, ptr["cen"], ids.ctypes.data, 1, 1, t, t, 32, nnz, ptr["pay"],
                                      ptr["bm"], t, None)
    assert rc == ERR_INVALID and b"x" in lib.reskv_last_error()


def test_operator_tables_refuse_tensors_of_another_device():
    import torch

    from reskv_b200._extension import _same_device, device_index_of

    assert device_index_of(torch.device("cuda", 3)) == 3 and device_index_of(2) == 2
    with pytest.raises(ValueError, match="must live on cuda:0"):
        _same_device(0, torch.zeros(1))
    _same_device(0, None)


def test_group_entry_points_check_their_arguments_before_any_launch():
    """``reskv_compress_group`` / ``reskv_window_shift``: null pointers, a group that does not fit the buffers, bad
    shift ranges and host memory are all refused with RESKV_ERR_INVALID (nothing is launched, so no GPU is needed)."""
    import numpy as np

    from reskv_b200._extension import ERR_INVALID, library

    lib = library()
    x = np.zeros((1, 64, 128), np.float16)
    cen = np.zeros((1, 8, 128), np.float16)
    ids = np.zeros((1, 256), np.int8)
    pay = np.zeros((1, 256, 32), np.float16)
    bm = np.zeros((1, 256, 2), np.int64)
    scratch = np.zeros((2, 1, 64), np.int32)
    p = lambda a: a.ctypes.data  # noqa: E731
    side = (p(cen), 8, p(cen), 8, p(ids), p(pay), p(bm), None)

    def group(seq_len, x_k=p(x), stride=256):
        return lib.reskv_compress_group(0, 16, 32, x_k, p(x), 1, 1, 64, 64, *side, stride, *side, stride, seq_len,
                                        p(scratch), None)

    assert group(0, x_k=None) == ERR_INVALID and b"null" in lib.reskv_last_error()
    assert group(200) == ERR_INVALID and b"do not fit" in lib.reskv_last_error()
    assert group(-1) == ERR_INVALID
    assert group(0) == ERR_INVALID and b"compress_group: k_ids" in lib.reskv_last_error()  # host pointers

    win = np.zeros((3, 1, 16, 128), np.float16)
    w = [p(win[i]) for i in range(3)]
    assert all(a % 16 == 0 for a in w)
    for dst, src, count in ((5, 4, 2), (0, 10, 7), (-1, 4, 2), (0, 4, -1)):
        assert lib.reskv_window_shift(*w, 1, 1, 16, dst, src, count, None) == ERR_INVALID
        assert b"window_shift" in lib.reskv_last_error()
    assert lib.reskv_window_shift(None, w[1], w[2], 1, 1, 16, 0, 4, 2, None) == ERR_INVALID
    assert lib.reskv_window_shift(*w, 1, 1, 16, 0, 4, 2, None) == ERR_INVALID  # host memory
    assert b"window_shift: window_k" in lib.reskv_last_error()

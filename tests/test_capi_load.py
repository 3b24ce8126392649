"""CPU tests: the C-ABI library loads, exports every declared symbol and rejects
bad arguments before touching a device."""
import ctypes as C
import importlib
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
capi = importlib.import_module("610sample_b200.capi")


def declared_symbols():
    with open(os.path.join(ROOT, "include", "attn_b200.h")) as f:
        text = f.read()
    return sorted(set(re.findall(r"\b(attn_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(capi.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(capi.EXPORTS)


def test_version_and_error_strings():
    lib = capi.lib()
    assert b"sm_100a" in lib.attn_b200_version()
    assert isinstance(lib.attn_b200_last_error(), bytes)


@pytest.mark.parametrize("field,value,code", [
    ("D", 72, -1), ("D", 0, -1), ("D", 256, -2), ("dtype", 7, -2), ("mask_mode", 3, -1),
    ("window_size", -1, -1), ("chunk_id", -2, -1), ("impl", 9, -1), ("N_q", -5, -1),
])
def test_shape_validation(field, value, code):
    lib = capi.lib()
    kw = dict(B=1, H=1, N_q=64, N_kv=64, D=64, window_size=64, chunk_id=0, mask_mode=0, dtype=capi.ATTN_BF16, impl=0)
    kw[field] = value
    s = capi.Shape(**kw)
    rc = lib.attn_b200_forward(s, 16, 16, 16, 16, 16, None)
    assert rc == code
    assert lib.attn_b200_last_error() != b""


def test_pointer_validation_and_unsupported_tensor_impl():
    lib = capi.lib()
    s = capi.make_shape(1, 1, 64, 64, 64, 64, 0, 0, capi.ATTN_BF16)
    assert lib.attn_b200_forward(s, None, 16, 16, 16, 16, None) == -1        # null pointer
    assert lib.attn_b200_forward(s, 8, 16, 16, 16, 16, None) == -1           # misaligned pointer
    assert lib.attn_b200_forward(None, 16, 16, 16, 16, 16, None) == -1       # null shape
    s = capi.make_shape(1, 1, 64, 64, 144, 64, 0, 0, capi.ATTN_BF16, capi.IMPL_TENSOR)
    assert lib.attn_b200_forward(s, 16, 16, 16, 16, 16, None) == -2          # head dimension above 128
    s = capi.make_shape(1, 1, 64, 64, 64, 64, 0, 0, capi.ATTN_F32, capi.IMPL_TENSOR)
    assert lib.attn_b200_forward(s, 16, 16, 16, 16, 16, None) == -2


def test_scratch_sizes_and_empty_problem():
    lib = capi.lib()
    s = capi.make_shape(2, 3, 100, 40, 64, 10, 0, 0, capi.ATTN_BF16)
    assert lib.attn_b200_backward_scratch_bytes(s) == 4 * 2 * 3 * 100
    assert lib.attn_b200_double_backward_scratch_bytes(s) == 3 * 4 * 2 * 3 * 100
    empty = capi.make_shape(0, 4, 64, 64, 64, 64, 0, 0, capi.ATTN_BF16)
    assert lib.attn_b200_forward(empty, 16, 16, 16, 16, 16, None) == 0       # nothing to do, no launch
    assert lib.attn_b200_last_launch_count() == 0
    assert lib.attn_b200_double_backward_phases(s, *([16] * 13), 16, None, 0) == -1
    assert lib.attn_b200_double_backward_phases(s, *([16] * 13), 16, None, 8) == -1

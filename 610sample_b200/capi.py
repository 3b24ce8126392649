"""ctypes binding of ``libattn_b200.so`` (``include/attn_b200.h``).

This is the stub a host program without PyTorch would write; the tests and the
bench use it to call the C ABI directly with raw device pointers.  Loading fails
loudly when the library has not been built -- there is no other code path.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libattn_b200.so")

ATTN_F16, ATTN_BF16, ATTN_F32 = 0, 1, 2
MASK_REFERENCE, MASK_NONE = 0, 1
IMPL_AUTO, IMPL_SIMT, IMPL_TENSOR = 0, 1, 2
ATTN_OK = 0
ATTN_ETOOLARGE = -5
STATIC_SCRATCH_ROWS = 1 << 20

EXPORTS = (
    "attn_b200_forward", "attn_b200_backward_scratch_bytes", "attn_b200_backward",
    "attn_b200_double_backward_scratch_bytes", "attn_b200_double_backward",
    "attn_b200_double_backward_phases", "attn_b200_double_backward_static",
    "attn_b200_last_launch_count", "attn_b200_device_status", "attn_b200_last_error",
    "attn_b200_version", "attn_b200_selftest_gemm", "attn_b200_set_status_mirror", "attn_b200_qk_norm_rope",
)


class Shape(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("B", "H", "N_q", "N_kv", "D", "window_size", "chunk_id", "mask_mode", "dtype", "impl")]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python 610sample_b200/_build.py`")
        L = C.CDLL(LIB_PATH)
        vp, fp = C.c_void_p, C.c_void_p
        L.attn_b200_forward.argtypes = [C.POINTER(Shape), vp, vp, vp, vp, fp, vp]
        L.attn_b200_backward_scratch_bytes.argtypes = [C.POINTER(Shape)]
        L.attn_b200_backward_scratch_bytes.restype = C.c_size_t
        L.attn_b200_backward.argtypes = [C.POINTER(Shape)] + [vp] * 9 + [fp, vp]
        L.attn_b200_double_backward_scratch_bytes.argtypes = [C.POINTER(Shape)]
        L.attn_b200_double_backward_scratch_bytes.restype = C.c_size_t
        L.attn_b200_double_backward.argtypes = [C.POINTER(Shape)] + [vp] * 13 + [fp, vp]
        L.attn_b200_double_backward_phases.argtypes = [C.POINTER(Shape)] + [vp] * 13 + [fp, vp, C.c_int32]
        L.attn_b200_double_backward_static.argtypes = [C.POINTER(Shape)] + [vp] * 13 + [vp]
        L.attn_b200_device_status.argtypes = [C.POINTER(C.c_uint32)]
        L.attn_b200_set_status_mirror.argtypes = [vp]
        L.attn_b200_qk_norm_rope.argtypes = [vp, vp, vp, vp] + [C.c_int32] * 5 + [C.c_float, C.c_int32, vp]
        L.attn_b200_last_error.restype = C.c_char_p
        L.attn_b200_version.restype = C.c_char_p
        L.attn_b200_selftest_gemm.argtypes = [vp, vp, fp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, vp]
        for name in EXPORTS:
            getattr(L, name)
        _lib = L
    return _lib


class AttnError(RuntimeError):
    def __init__(self, what: str, code: int):
        msg = lib().attn_b200_last_error().decode()
        super().__init__(f"{what} failed ({code}): {msg}")
        self.code = code


def check(code: int, what: str) -> None:
    if code != ATTN_OK:
        raise AttnError(what, code)


def make_shape(B, H, N_q, N_kv, D, window_size, chunk_id, mask_mode, dtype, impl=IMPL_AUTO) -> Shape:
    return Shape(B, H, N_q, N_kv, D, window_size, chunk_id, mask_mode, dtype, impl)


def device_status() -> int:
    code = C.c_uint32(0)
    rc = lib().attn_b200_device_status(C.byref(code))
    if rc not in (ATTN_OK, -4):
        raise AttnError("attn_b200_device_status", rc)
    return int(code.value)

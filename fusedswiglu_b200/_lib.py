"""ctypes binding of the C ABI declared in include/fused_swiglu.h.

The shared library is the only compute path: if it is missing or a call fails,
an exception is raised.  There is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_uint32, c_uint64, c_void_p, POINTER
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libfused_swiglu_sm100.so"

FSW_BF16, FSW_FP16 = 0, 1
FSW_ACC_F32, FSW_ACC_F16 = 0, 1
FSW_OK = 0

# name -> (restype, argtypes); mirrors include/fused_swiglu.h one to one.
SIGNATURES = {
    "fsw_forward": (c_int, [c_void_p] * 6 + [c_int64] * 3 + [c_int, c_int, c_void_p]),
    "fsw_backward_elementwise": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_void_p]),
    "fsw_backward_dx": (c_int, [c_void_p] * 5 + [c_int64] * 3 + [c_int, c_int, c_void_p]),
    "fsw_backward_dx_scatter": (c_int, [c_void_p] * 4 + [POINTER(c_void_p), c_int, c_int] + [c_int64] * 3 + [c_int, c_int, c_void_p]),
    "fsw_dx_reduce": (c_int, [c_void_p, c_void_p, POINTER(c_void_p), c_void_p, c_int, c_int, c_uint32, c_int64, c_int64, c_void_p, c_int, c_void_p]),
    "fsw_wait_flags": (c_int, [c_void_p, c_int, c_uint32, c_void_p]),
    "fsw_backward_dw": (c_int, [c_void_p] * 5 + [c_int64] * 3 + [c_int, c_int, c_void_p]),
    "fsw_backward_dw_columns": (c_int, [c_void_p] * 5 + [c_int64] * 5 + [c_int, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "fsw_forward_ws": (c_int, [c_void_p] * 6 + [c_int64] * 3 + [c_void_p, c_int64, c_int, c_int, c_void_p]),
    "fsw_forward_st": (c_int, [c_void_p] * 6 + [c_int64] * 3 + [c_int, c_int, c_void_p]),
    "fsw_backward_dx_fused": (c_int, [c_void_p] * 8 + [c_int64] * 3 + [c_int, c_void_p]),
    "fsw_backward_elementwise_st": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_void_p]),
    "fsw_backward_dx_gate": (c_int, [c_void_p] * 8 + [c_int64] * 3 + [c_void_p, c_int64, c_int, c_void_p]),
    "fsw_backward_dx_ws": (c_int, [c_void_p] * 5 + [c_int64] * 3 + [c_void_p, c_int64, c_int, c_int, c_void_p]),
    "fsw_workspace_bytes": (c_int64, []),
    "fsw_backward": (c_int, [c_void_p] * 11 + [c_int64] * 3 + [c_int, c_int, c_void_p]),
    "fsw_gemm": (c_int, [c_void_p] * 3 + [c_int64] * 3 + [c_int] * 4 + [c_void_p]),
    "fsw_gemm_ws": (c_int, [c_void_p] * 3 + [c_int64] * 3 + [c_int, c_int, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "fsw_backward_static_scratch": (c_int, [c_void_p] * 9 + [c_int64] * 3 + [c_int, c_int, c_void_p]),
    "fsw_debug_split_work": (c_int, [c_int] * 7 + [POINTER(c_int64), POINTER(c_int)]),
    "fsw_debug_decode_tile": (c_int, [c_int] * 4 + [POINTER(c_int), POINTER(c_int)]),
    "fsw_debug_descriptors": (c_int, [c_int] * 6 + [POINTER(c_uint32), POINTER(c_uint64), POINTER(c_uint64)]),
    "fsw_last_error": (c_char_p, []),
    "fsw_query_device": (c_int, [c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int64)]),
    "fsw_status": (c_int64, []),
    "fsw_set_option": (c_int, [c_char_p, c_int64]),
    "fsw_get_option": (c_int64, [c_char_p]),
}

_lib = None


class FusedSwiGLUError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, code: int, message: str):
        super().__init__(f"{fn} failed with code {code}: {message}")
        self.code = code


def load() -> ctypes.CDLL:
    """Load the library once and declare every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing. Build it with `python -m fusedswiglu_b200.build` "
            "(needs nvcc). This package has no fallback path."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return (load().fsw_last_error() or b"").decode()


def check(fn: str, code: int) -> None:
    if code != FSW_OK:
        raise FusedSwiGLUError(fn, code, last_error())


def set_option(name: str, value: int) -> None:
    check("fsw_set_option", load().fsw_set_option(name.encode(), int(value)))


def get_option(name: str) -> int:
    return int(load().fsw_get_option(name.encode()))


def device_status() -> int:
    """Synchronise and return the kernels' status word (0 = every wait completed)."""
    v = int(load().fsw_status())
    if v < 0:
        raise FusedSwiGLUError("fsw_status", v, last_error())
    return v

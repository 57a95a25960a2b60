"""The C-ABI shared library loads without a GPU and exports exactly what
include/fused_swiglu.h declares; argument checking works before any CUDA call."""
import ctypes
import re
from pathlib import Path

import pytest

from fusedswiglu_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "fused_swiglu.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(fsw_[a-z_0-9]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for required in ("fsw_forward", "fsw_backward_elementwise", "fsw_backward_dx", "fsw_backward_dw",
                     "fsw_backward", "fsw_last_error", "fsw_query_device", "fsw_status"):
        assert required in names


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(str(built_library))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_table_covers_the_header():
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_header_has_no_torch_or_cxx_types():
    text = HEADER.read_text()
    assert "torch" not in text.lower() and "std::" not in text and "at::" not in text
    assert 'extern "C"' in text


def test_argument_errors_are_reported_not_raised_across_the_abi():
    lib = _lib.load()
    # dtype 7 does not exist
    rc = lib.fsw_forward(None, None, None, None, None, None, 8, 64, 64, 7, 0, None)
    assert rc == -1 and "dtype" in _lib.last_error()
    # d_model not a multiple of 8
    rc = lib.fsw_forward(None, None, None, None, None, None, 8, 60, 64, 0, 0, None)
    assert rc == -1 and "multiples of 8" in _lib.last_error()
    # fp16 accumulation with bf16 tensors
    rc = lib.fsw_backward_dw(None, None, None, None, None, 8, 64, 64, 0, 1, None)
    assert rc == -1 and "fp16" in _lib.last_error()
    # NULL tensors
    rc = lib.fsw_forward(None, None, None, None, None, None, 8, 64, 64, 0, 0, None)
    assert rc == -1 and "required" in _lib.last_error()
    # column range outside the array, or not a multiple of 8
    rc = lib.fsw_backward_dw_columns(None, None, None, None, None, 8, 64, 64, 32, 40, 0, 0, 0, None)
    assert rc == -1 and "column range" in _lib.last_error()
    rc = lib.fsw_backward_dw_columns(None, None, None, None, None, 8, 64, 64, 4, 8, 0, 0, 0, None)
    assert rc == -1 and "column range" in _lib.last_error()
    # a negative SM cap
    rc = lib.fsw_backward_dw_columns(None, None, None, None, None, 8, 64, 64, 0, 8, -1, 0, 0, None)
    assert rc == -1 and "max_sms" in _lib.last_error()
    # misaligned pointer
    rc = lib.fsw_backward_elementwise(8, 16, 16, 16, 16, 64, 0, None)
    assert rc == -1 and "aligned" in _lib.last_error()
    with pytest.raises(_lib.FusedSwiGLUError):
        _lib.check("fsw_forward", rc)


def test_options_roundtrip():
    old = _lib.get_option("group_m")
    _lib.set_option("group_m", 4)
    assert _lib.get_option("group_m") == 4
    _lib.set_option("group_m", old)
    with pytest.raises(_lib.FusedSwiGLUError):
        _lib.set_option("cta_group", 3)
    with pytest.raises(_lib.FusedSwiGLUError):
        _lib.set_option("no_such_option", 1)
    assert _lib.get_option("no_such_option") == -1
    # bounds of the device-wait limit and of the automatic settings
    assert _lib.get_option("wait_limit_ms") == 2000
    with pytest.raises(_lib.FusedSwiGLUError):
        _lib.set_option("wait_limit_ms", 0)
    for name in ("cta_group", "nsub", "group_m"):
        assert _lib.get_option(name) == 0  # 0 = chosen per launch
    with pytest.raises(_lib.FusedSwiGLUError):
        _lib.set_option("nsub", 3)


def test_tile_rasterisation_visits_every_tile_exactly_once():
    """The grouped tile order used by the kernels is a permutation of the tile grid
    for ragged group sizes too, and walks group_m rows before the column advances."""
    lib = _lib.load()
    m, n = ctypes.c_int(), ctypes.c_int()
    for num_m, num_n, gm in [(1, 1, 1), (5, 3, 2), (7, 4, 16), (16, 56, 16), (128, 8, 2), (33, 9, 8), (3, 1, 5)]:
        seen = []
        for t in range(num_m * num_n):
            assert lib.fsw_debug_decode_tile(t, num_m, num_n, gm, ctypes.byref(m), ctypes.byref(n)) == 0
            assert 0 <= m.value < num_m and 0 <= n.value < num_n
            seen.append((m.value, n.value))
        assert len(set(seen)) == num_m * num_n, (num_m, num_n, gm)
        # the first min(gm, num_m) tiles share column 0 and have consecutive rows
        first = min(gm, num_m)
        assert seen[:first] == [(i, 0) for i in range(first)]
    assert lib.fsw_debug_decode_tile(99, 3, 3, 1, ctypes.byref(m), ctypes.byref(n)) == -1


def test_descriptor_encoders_known_answers():
    """Bit layouts of the tcgen05 descriptors, checked against values assembled by
    hand from the documented fields.  Instruction descriptor (kind::f16): D format
    at bit 4 (1 = fp32), A/B format at bits 7/10 (1 = bf16, 0 = fp16), A/B major at
    bits 15/16 (1 = MN-major), N>>3 at bit 17, M>>4 at bit 24.  Shared-memory
    descriptor: leading byte offset >>4 at bit 16, stride byte offset >>4 at bit 32,
    version 1 at bit 46, layout type 2 (128-byte swizzle) at bit 61."""
    lib = _lib.load()
    idesc, sk, smn = ctypes.c_uint32(), ctypes.c_uint64(), ctypes.c_uint64()

    def q(dtype, accum, a_major, b_major, m, n):
        assert lib.fsw_debug_descriptors(dtype, accum, a_major, b_major, m, n, ctypes.byref(idesc),
                                         ctypes.byref(sk), ctypes.byref(smn)) == 0
        return idesc.value

    # forward: bf16, fp32 acc, A K-major, B MN-major, CTA pair M=256, N=256
    assert q(0, 0, 0, 1, 256, 256) == (1 << 4) | (1 << 7) | (1 << 10) | (1 << 16) | (32 << 17) | (16 << 24)
    # dX: both K-major
    assert q(0, 0, 0, 0, 256, 256) == (1 << 4) | (1 << 7) | (1 << 10) | (32 << 17) | (16 << 24)
    # dW: both MN-major, single CTA M=128
    assert q(0, 0, 1, 1, 128, 256) == (1 << 4) | (1 << 7) | (1 << 10) | (3 << 15) | (32 << 17) | (8 << 24)
    # fp16 with fp16 accumulator: all format fields zero
    assert q(1, 1, 0, 1, 256, 256) == (1 << 16) | (32 << 17) | (16 << 24)
    # K-major: LBO 16 B (ignored with swizzle), SBO 1024 B; MN-major: LBO 8192 B, SBO 1024 B
    assert sk.value == (1 << 16) | (64 << 32) | (1 << 46) | (2 << 61)
    assert smn.value == (512 << 16) | (64 << 32) | (1 << 46) | (2 << 61)
    assert lib.fsw_debug_descriptors(5, 0, 0, 0, 128, 256, ctypes.byref(idesc), ctypes.byref(sk), ctypes.byref(smn)) == -1

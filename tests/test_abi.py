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
    rc = lib.fsw_backward_dw_columns(None, None, None, None, None, 8, 64, 64, 32, 40, 0, None, 0, 0, 0, None)
    assert rc == -1 and "column range" in _lib.last_error()
    rc = lib.fsw_backward_dw_columns(None, None, None, None, None, 8, 64, 64, 4, 8, 0, None, 0, 0, 0, None)
    assert rc == -1 and "column range" in _lib.last_error()
    # a negative SM cap
    rc = lib.fsw_backward_dw_columns(None, None, None, None, None, 8, 64, 64, 0, 8, -1, None, 0, 0, 0, None)
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


def test_split_of_the_last_wave_covers_every_k_iteration_exactly_once():
    """Host copy of the kernels' work distribution: whole tiles in full waves, then the
    K iterations of the remaining tiles cut into equal shares, one per SM pair.  Every
    (tile, K iteration) must be computed exactly once, a pair touches at most two split
    tiles, slots are unique, and the pieces of a tile are found by the rule the second
    kernel uses (pair c's first piece belongs to tile floor(c * share / iterations))."""
    lib = _lib.load()
    plan = (ctypes.c_int64 * 3)()
    item = (ctypes.c_int * 6)()
    cases = [  # (m tiles, n tiles, group_m, K iterations per tile, SM pairs), expect split
        ((16, 56, 16, 512, 74), True),    # dW of the Llama-3-8B shape: 12 waves + 8 tiles
        ((16, 7, 16, 512, 74), True),     # its 1/8 column shard: 1 wave + 38 tiles
        ((16, 7, 2, 512, 66), True),      # the same on 132 SMs: 1 wave + 46 tiles
        ((16, 7, 2, 512, 58), False),     # on 116 SMs: 1 wave + 54 of 58, nothing to gain
        ((4, 10, 4, 256, 74), True),      # fewer tiles than pairs
        ((128, 8, 2, 448, 74), False),    # dX of the same shape: 13 waves + 62 of 74, nothing to gain
        ((24, 4, 2, 150, 74), True),      # a dX with 1 wave + 22 tiles
        ((2, 37, 2, 300, 74), False),     # a whole number of waves
        ((1, 3, 1, 2, 74), False),        # K too short to be worth a second kernel
        ((3, 5, 2, 1000, 7), True),
    ]
    for (nm, nn, gm, ipt, pairs), expect in cases:
        rc = lib.fsw_debug_split_work(nm, nn, gm, ipt, pairs, 0, 0, plan, None)
        assert rc == (1 if expect else 0), (nm, nn, ipt, pairs, rc)
        first_tile, share, total = plan[0], plan[1], plan[2]
        tiles = nm * nn
        if expect:
            assert first_tile % pairs == 0 and 0 < tiles - first_tile < pairs
            assert total == (tiles - first_tile) * ipt and share * pairs >= total > share * (pairs - 1) - share
        covered = {}
        slots = set()
        order = []
        for c in range(pairs):
            pieces = 0
            for idx in range(tiles // pairs + 4):
                assert lib.fsw_debug_split_work(nm, nn, gm, ipt, pairs, c, idx, plan, item) >= 0
                if not item[0]:
                    continue
                m, n, it0, it1, slot = item[1], item[2], item[3], item[4], item[5]
                assert 0 <= m < nm and 0 <= n < nn and 0 <= it0 < it1 <= ipt
                for it in range(it0, it1):
                    assert (m, n, it) not in covered, (c, idx, m, n, it)
                    covered[(m, n, it)] = slot
                if slot >= 0:
                    pieces += 1
                    assert slot not in slots and slot == 2 * c + (pieces - 1)
                    slots.add(slot)
                    order.append((m, n, it0, c, slot))
                else:
                    assert (it0, it1) == (0, ipt)
            assert pieces <= 2
        assert len(covered) == tiles * ipt, (nm, nn, ipt, pairs)
        # the second kernel's rule for finding the pieces of split tile j, in K order
        if expect:
            m_, n_ = ctypes.c_int(), ctypes.c_int()
            for j in range(tiles - first_tile):
                lib.fsw_debug_decode_tile(first_tile + j, nm, nn, gm, ctypes.byref(m_), ctypes.byref(n_))
                c_lo, c_hi = (j * ipt) // share, ((j + 1) * ipt - 1) // share
                want = [2 * c + (0 if (c * share) // ipt == j else 1) for c in range(c_lo, c_hi + 1)]
                have = [s for (m, n, it0, c, s) in sorted(order, key=lambda o: (o[0], o[1], o[2]))
                        if (m, n) == (m_.value, n_.value)]
                assert have == want, (j, have, want)


def test_argument_errors_of_the_multi_gpu_and_fused_entry_points():
    lib = _lib.load()
    P = ctypes.c_void_p
    two = (P * 2)(P(16), P(32))
    # world size outside 2..8, and T that does not split into rows that are multiples of 32
    assert lib.fsw_backward_dx_scatter(P(16), P(16), P(16), P(16), two, 1, 0, 64, 64, 64, 0, 0, None) == -1
    assert "world size" in _lib.last_error()
    assert lib.fsw_backward_dx_scatter(P(16), P(16), P(16), P(16), two, 2, 0, 80, 64, 64, 0, 0, None) == -1
    assert "multiple of 32" in _lib.last_error()
    # reduction: rank outside the world, misaligned buffers
    assert lib.fsw_dx_reduce(P(16), None, two, P(16), 2, 2, 1, 32, 64, P(16), 0, None) == -1
    assert "rank" in _lib.last_error()
    assert lib.fsw_dx_reduce(P(8), None, two, P(16), 2, 0, 1, 32, 64, P(16), 0, None) == -1
    assert "aligned" in _lib.last_error()
    assert lib.fsw_wait_flags(None, 2, 1, None) == -1
    # fused gate gradient: every pointer is required, numel of the elementwise form a multiple of 8
    assert lib.fsw_backward_dx_fused(P(16), None, P(16), P(16), P(16), P(16), P(16), P(16), 64, 64, 64, 0, None) == -1
    assert "NULL" in _lib.last_error()
    assert lib.fsw_backward_elementwise_st(P(16), P(16), P(16), P(16), P(16), 12, 0, None) == -1
    assert lib.fsw_forward_st(P(16), P(16), P(16), P(16), None, None, 64, 64, 64, 0, 0, None) == -1
    # workspace size must not be negative
    assert lib.fsw_backward_dw_columns(P(16), P(16), P(16), P(16), P(16), 8, 64, 64, 0, 8, 0, None, -1, 0, 0, None) == -1

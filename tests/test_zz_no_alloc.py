"""The allocation-free backward entry point, fsw_backward_static_scratch.

It serves hosts that cannot allocate device memory where they call the backward
(fixed memory plans, plugin enqueue hooks, loops that cannot tolerate the
synchronisation of cudaMalloc): its dg/du scratch is a fixed array inside the
library.  The tests drive it through the C ABI, several calls in a row with
different inputs, and require each result to be bit-identical to fsw_backward
given torch-allocated scratch (the two run the same kernels on the same inputs).
This file is collected last so that a failure here cannot mask any other test.
"""
import ctypes
import math

import pytest
import torch

from fusedswiglu_b200 import _lib

LIMIT = 4 * 1024 * 1024  # FSW_STATIC_SCRATCH_ELEMS in include/fused_swiglu.h
DT = {0: torch.bfloat16, 1: torch.float16}


def test_sizes_beyond_the_built_in_scratch_are_rejected():
    lib = _lib.load()
    T, dm, di = 2048, 64, 4096  # T*di = 8 Mi elements > 4 Mi
    assert T * di > LIMIT
    rc = lib.fsw_backward_static_scratch(None, None, None, None, None, None, None, None, None,
                                         T, dm, di, 0, 0, None)
    assert rc == -1
    msg = _lib.last_error()
    assert "exceeds the built-in scratch" in msg and str(LIMIT) in msg
    # the first size above the limit (T*di = 4 Mi + 8) is refused too
    T, di = 1, LIMIT + 8
    rc = lib.fsw_backward_static_scratch(None, None, None, None, None, None, None, None, None,
                                         T, dm, di, 0, 0, None)
    assert rc == -1 and "exceeds the built-in scratch" in _lib.last_error()


def _case(lib, st, seed, T, dm, di, dtype):
    """One forward, then the backward through both entry points; returns (got, ref)."""
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    tdt = DT[dtype]
    gen = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", dtype=tdt, generator=gen)
    x, dout = mk(T, dm), mk(T, di)
    wg, wu = mk(dm, di) / math.sqrt(dm), mk(dm, di) / math.sqrt(dm)
    out, g, u = (torch.empty(T, di, device="cuda", dtype=tdt) for _ in range(3))
    _lib.check("fsw_forward", lib.fsw_forward(p(x), p(wg), p(wu), p(out), p(g), p(u), T, dm, di, dtype, 0, st))
    shapes = (("dx", (T, dm)), ("dwg", (dm, di)), ("dwu", (dm, di)))
    ref = {k: torch.empty(s, device="cuda", dtype=tdt) for k, s in shapes}
    got = {k: torch.full(s, float("nan"), device="cuda", dtype=tdt) for k, s in shapes}
    dg, du = torch.empty_like(out), torch.empty_like(out)
    _lib.check("fsw_backward", lib.fsw_backward(
        p(dout), p(x), p(wg), p(wu), p(g), p(u), p(dg), p(du), p(ref["dx"]), p(ref["dwg"]), p(ref["dwu"]),
        T, dm, di, dtype, 0, st))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]  # cudaMemGetInfo: every output exists by now
    _lib.check("fsw_backward_static_scratch", lib.fsw_backward_static_scratch(
        p(dout), p(x), p(wg), p(wu), p(g), p(u), p(got["dx"]), p(got["dwg"]), p(got["dwu"]),
        T, dm, di, dtype, 0, st))
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    return got, ref, free_before - free_after


@pytest.mark.gpu
def test_calls_in_a_row_are_bit_identical_to_the_caller_scratch_entry_point():
    assert torch.cuda.is_available()
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    cases = [
        (1024, 512, 2048, 0),   # first call on the device: resolves the array's address
        (384, 256, 1280, 0),    # smaller: stale dg/du of the call before stay beyond what this one writes
        (1024, 64, 4096, 0),    # T*di == the limit exactly: du ends on the array's last byte
        (100, 72, 136, 0),      # T*di*2 bytes is not a multiple of 256: du starts on the next boundary
        (512, 256, 1024, 1),    # fp16
    ]
    for seed, (T, dm, di, dtype) in enumerate(cases):
        assert T * di <= LIMIT
        got, ref, leaked = _case(lib, st, seed, T, dm, di, dtype)
        for k in ref:
            assert torch.equal(got[k], ref[k]), (seed, k)
        if seed > 0:
            # nothing was allocated by the call (the first call may have made the
            # CUDA module's one-time set-up; later ones must not move the free count)
            assert leaked == 0, (seed, leaked)
    assert (1024 * 4096 == LIMIT) and (100 * 136 * 2) % 256 != 0
    assert _lib.device_status() == 0

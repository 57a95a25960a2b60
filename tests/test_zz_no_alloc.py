"""The allocation-free backward entry point, fsw_backward_static_scratch.

It serves hosts that cannot allocate device memory where they call the backward
(fixed memory plans, plugin enqueue hooks, loops that cannot tolerate the
synchronisation of cudaMalloc): its dg/du scratch is a fixed array inside the
library.  The test drives it through the C ABI twice in a row with different
inputs and checks each result against fsw_backward given torch-allocated scratch.
This file is collected last so that a failure here cannot mask any other test.
"""
import ctypes
import math

import pytest
import torch

from fusedswiglu_b200 import _lib

LIMIT = 4 * 1024 * 1024  # FSW_STATIC_SCRATCH_ELEMS in include/fused_swiglu.h
TOL = 1e-2               # the relative-Frobenius bound used throughout the GPU tests


def test_sizes_beyond_the_built_in_scratch_are_rejected():
    lib = _lib.load()
    T, dm, di = 2048, 64, 4096  # T*di = 8 Mi elements > 4 Mi
    assert T * di > LIMIT
    rc = lib.fsw_backward_static_scratch(None, None, None, None, None, None, None, None, None,
                                         T, dm, di, 0, 0, None)
    assert rc == -1
    msg = _lib.last_error()
    assert "exceeds the built-in scratch" in msg and str(LIMIT) in msg


def _rel(a, b):
    return (torch.linalg.norm(a.float() - b.float()) / torch.linalg.norm(b.float())).item()


@pytest.mark.gpu
def test_two_calls_in_a_row_match_the_caller_scratch_entry_point():
    assert torch.cuda.is_available()
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    # second call is smaller than the first, so stale dg/du from call 1 stay in the
    # array beyond what call 2 writes
    for seed, (T, dm, di) in enumerate([(1024, 512, 2048), (384, 256, 1280)]):
        assert T * di <= LIMIT
        gen = torch.Generator(device="cuda").manual_seed(seed)
        mk = lambda *s: torch.randn(*s, device="cuda", dtype=torch.bfloat16, generator=gen)
        x, dout = mk(T, dm), mk(T, di)
        wg, wu = mk(dm, di) / math.sqrt(dm), mk(dm, di) / math.sqrt(dm)
        out, g, u = (torch.empty(T, di, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        _lib.check("fsw_forward", lib.fsw_forward(p(x), p(wg), p(wu), p(out), p(g), p(u), T, dm, di, 0, 0, st))

        ref = {k: torch.empty(s, device="cuda", dtype=torch.bfloat16)
               for k, s in (("dx", (T, dm)), ("dwg", (dm, di)), ("dwu", (dm, di)))}
        dg, du = torch.empty_like(out), torch.empty_like(out)
        _lib.check("fsw_backward", lib.fsw_backward(
            p(dout), p(x), p(wg), p(wu), p(g), p(u), p(dg), p(du), p(ref["dx"]), p(ref["dwg"]), p(ref["dwu"]),
            T, dm, di, 0, 0, st))

        got = {k: torch.full_like(v, float("nan")) for k, v in ref.items()}
        _lib.check("fsw_backward_static_scratch", lib.fsw_backward_static_scratch(
            p(dout), p(x), p(wg), p(wu), p(g), p(u), p(got["dx"]), p(got["dwg"]), p(got["dwu"]),
            T, dm, di, 0, 0, st))
        torch.cuda.synchronize()
        for k in ref:
            assert torch.all(torch.isfinite(got[k].float())), k
            err = _rel(got[k], ref[k])
            assert err < TOL, (seed, k, err)
    assert _lib.device_status() == 0

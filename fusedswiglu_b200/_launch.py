"""Host launchers: torch tensors in, C-ABI calls out.

torch is used only for device memory, the current stream and dtype bookkeeping;
every arithmetic result comes from libfused_swiglu_sm100.so.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

_DTYPE_CODE = {torch.bfloat16: _lib.FSW_BF16, torch.float16: _lib.FSW_FP16}


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise AssertionError(f"Expected torch.bfloat16 or torch.float16 tensors, got {t.dtype}") from None


def _require_cuda(*tensors: torch.Tensor) -> None:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError(
                "fused_swiglu runs on CUDA tensors only (sm_100a); there is no CPU path"
            )
        if t.device != dev:
            raise RuntimeError(f"all tensors must be on one device, got {dev} and {t.device}")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


_WORKSPACE_BYTES = {}
_WORKSPACES = {}


def _workspace(t: torch.Tensor) -> Optional[torch.Tensor]:
    """Scratch for the split of a GEMM's last wave of tiles along K (see
    fsw_workspace_bytes in the header): one buffer per (device, stream), allocated by
    torch on first use and kept.  Launches on one stream run in order, so they can share
    it; launches on different streams, which may overlap, get different buffers.  The
    library itself allocates nothing."""
    dev = t.device.index
    if dev not in _WORKSPACE_BYTES:
        with torch.cuda.device(t.device):
            n = int(_lib.load().fsw_workspace_bytes())
        if n < 0:
            _lib.check("fsw_workspace_bytes", n)
        _WORKSPACE_BYTES[dev] = n
    key = (dev, torch.cuda.current_stream(t.device).cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            return None  # no allocation inside a graph capture: the launch just does not split
        ws = _WORKSPACES[key] = torch.empty(_WORKSPACE_BYTES[dev], device=t.device, dtype=torch.uint8)
    return ws


def forward(
    x2d: torch.Tensor,
    w_gate: torch.Tensor,
    w_up: torch.Tensor,
    *,
    fast_accum: bool = False,
    save_activations: bool = True,
    split_k: bool = True,
    save_factors: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """out, g, u for x2d (T, dm) and weights (dm, di); g and u are None when not saved.
    ``split_k`` lets the last partial wave of tiles be divided along K (needs scratch).
    ``save_factors``: return (out, s, t) with s = silu(g) and t = u * silu'(g), the two
    factors the fused backward multiplies dout by, instead of g and u."""
    if save_factors:
        _require_cuda(x2d, w_gate, w_up)
        T, dm = x2d.shape
        di = w_gate.shape[1]
        out = torch.empty((T, di), device=x2d.device, dtype=x2d.dtype)
        s, t = torch.empty_like(out), torch.empty_like(out)
        with torch.cuda.device(x2d.device):
            rc = _lib.load().fsw_forward_st(
                x2d.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), out.data_ptr(), s.data_ptr(), t.data_ptr(),
                T, dm, di, _code(x2d), _lib.FSW_ACC_F16 if fast_accum else _lib.FSW_ACC_F32, _stream(x2d))
        _lib.check("fsw_forward_st", rc)
        return out, s, t
    _require_cuda(x2d, w_gate, w_up)
    T, dm = x2d.shape
    di = w_gate.shape[1]
    out = torch.empty((T, di), device=x2d.device, dtype=x2d.dtype)
    g = torch.empty_like(out) if save_activations else None
    u = torch.empty_like(out) if save_activations else None
    ws = _workspace(x2d) if split_k and T > 0 else None
    with torch.cuda.device(x2d.device):
        rc = _lib.load().fsw_forward_ws(
            x2d.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), out.data_ptr(),
            g.data_ptr() if g is not None else None,
            u.data_ptr() if u is not None else None,
            T, dm, di, ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            _code(x2d), _lib.FSW_ACC_F16 if fast_accum else _lib.FSW_ACC_F32, _stream(x2d),
        )
    _lib.check("fsw_forward_ws", rc)
    return out, g, u


def gate_grad(dout: torch.Tensor, g: torch.Tensor, u: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(dg, du) from contiguous dout, g, u of one shape."""
    _require_cuda(dout, g, u)
    dg = torch.empty_like(dout)
    du = torch.empty_like(dout)
    with torch.cuda.device(dout.device):
        rc = _lib.load().fsw_backward_elementwise(
            dout.data_ptr(), g.data_ptr(), u.data_ptr(), dg.data_ptr(), du.data_ptr(),
            dout.numel(), _code(dout), _stream(dout),
        )
    _lib.check("fsw_backward_elementwise", rc)
    return dg, du


def grad_input(dg: torch.Tensor, du: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, *,
               split_k: bool = True) -> torch.Tensor:
    """dX (T, dm) = dg @ w_gate^T + du @ w_up^T, accumulated in fp32 in one GEMM.
    ``split_k`` lets the last partial wave of tiles be divided along K (needs scratch)."""
    _require_cuda(dg, du, w_gate, w_up)
    T, di = dg.shape
    dm = w_gate.shape[0]
    dx = torch.empty((T, dm), device=dg.device, dtype=dg.dtype)
    ws = _workspace(dg) if split_k and T > 0 else None
    with torch.cuda.device(dg.device):
        rc = _lib.load().fsw_backward_dx_ws(
            dg.data_ptr(), du.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), dx.data_ptr(),
            T, dm, di, ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            _code(dg), _lib.FSW_ACC_F32, _stream(dg),
        )
    _lib.check("fsw_backward_dx_ws", rc)
    return dx


def grad_weights(
    x2d: torch.Tensor, dg: torch.Tensor, du: torch.Tensor, *, fast_accum: bool = False,
    out_gate: Optional[torch.Tensor] = None, out_up: Optional[torch.Tensor] = None,
    columns: Optional[Tuple[int, int]] = None, max_sms: int = 0, split_k: bool = True,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """(dW_gate, dW_up), each (dm, di), reduced over all T rows of x2d.

    ``columns=(first, count)`` computes only that column range of both gradients
    (the rest of the output tensors is left as it is); pass ``out_gate``/``out_up``
    to collect several ranges in one pair of tensors.  ``max_sms`` > 0 caps the SMs
    this launch occupies (to leave room for a kernel that runs beside it).  ``split_k``
    lets the last partial wave of tiles be divided along the token dimension over all
    SMs (needs scratch; the sum is then associated differently in those tiles)."""
    _require_cuda(x2d, dg, du)
    T, dm = x2d.shape
    di = dg.shape[1]
    dwg = out_gate if out_gate is not None else torch.empty((dm, di), device=x2d.device, dtype=x2d.dtype)
    dwu = out_up if out_up is not None else torch.empty((dm, di), device=x2d.device, dtype=x2d.dtype)
    acc = _lib.FSW_ACC_F16 if fast_accum else _lib.FSW_ACC_F32
    with torch.cuda.device(x2d.device):
        ws = _workspace(x2d) if split_k and T > 0 else None
        if columns is None and (max_sms > 0 or ws is not None):
            columns = (0, di)
        if columns is None:
            name = "fsw_backward_dw"
            rc = _lib.load().fsw_backward_dw(
                x2d.data_ptr(), dg.data_ptr(), du.data_ptr(), dwg.data_ptr(), dwu.data_ptr(),
                T, dm, di, _code(x2d), acc, _stream(x2d),
            )
        else:
            name = "fsw_backward_dw_columns"
            rc = _lib.load().fsw_backward_dw_columns(
                x2d.data_ptr(), dg.data_ptr(), du.data_ptr(), dwg.data_ptr(), dwu.data_ptr(),
                T, dm, di, int(columns[0]), int(columns[1]), int(max_sms),
                ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                _code(x2d), acc, _stream(x2d),
            )
    _lib.check(name, rc)
    return dwg, dwu


def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
         fast_accum: bool = False, split_k: bool = True) -> torch.Tensor:
    """C = op(A) @ op(B) for contiguous 2-D 16-bit tensors: A (M,K) or, with trans_a,
    (K,M); B (K,N) or, with trans_b, (N,K).  fp32 accumulation unless fast_accum (fp16)."""
    _require_cuda(a, b)
    assert a.ndim == 2 and b.ndim == 2 and a.dtype == b.dtype, "Expected two 2-D tensors of one dtype"
    assert not (trans_a and trans_b), "A^T @ B^T is not provided"
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    Kb, N = (b.shape[1], b.shape[0]) if trans_b else b.shape
    assert K == Kb, f"Dimension mismatch. Expected inner sizes to agree, got {K} and {Kb}"
    c = torch.empty((M, N), device=a.device, dtype=a.dtype)
    ws = _workspace(a) if split_k and M > 0 and K > 0 else None
    with torch.cuda.device(a.device):
        rc = _lib.load().fsw_gemm_ws(
            a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, int(trans_a), int(trans_b),
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, _code(a),
            _lib.FSW_ACC_F16 if fast_accum else _lib.FSW_ACC_F32, _stream(a),
        )
    _lib.check("fsw_gemm_ws", rc)
    return c


def grad_input_fused(dout: torch.Tensor, s: torch.Tensor, t: torch.Tensor, w_gate: torch.Tensor,
                     w_up: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(dX, dg, du) in one launch from dout and the factors saved by
    ``forward(save_factors=True)``: dg = dout * t and du = dout * s are produced inside
    the dX GEMM and also written out for the weight-gradient GEMM."""
    _require_cuda(dout, s, t, w_gate, w_up)
    T, di = dout.shape
    dm = w_gate.shape[0]
    dx = torch.empty((T, dm), device=dout.device, dtype=dout.dtype)
    dg, du = torch.empty_like(dout), torch.empty_like(dout)
    with torch.cuda.device(dout.device):
        rc = _lib.load().fsw_backward_dx_fused(
            dout.data_ptr(), s.data_ptr(), t.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), dx.data_ptr(),
            dg.data_ptr(), du.data_ptr(), T, dm, di, _code(dout), _stream(dout))
    _lib.check("fsw_backward_dx_fused", rc)
    return dx, dg, du


def gate_grad_and_input(dout: torch.Tensor, g: torch.Tensor, u: torch.Tensor, w_gate: torch.Tensor,
                        w_up: torch.Tensor, *, split_k: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(dX, dg, du) in one launch: the gate-gradient step runs inside the dX GEMM kernel, on
    its otherwise idle epilogue warps (bit-identical to gate_grad + grad_input)."""
    _require_cuda(dout, g, u, w_gate, w_up)
    T, di = dout.shape
    dm = w_gate.shape[0]
    dx = torch.empty((T, dm), device=dout.device, dtype=dout.dtype)
    dg, du = torch.empty_like(dout), torch.empty_like(dout)
    ws = _workspace(dout) if split_k and T > 0 else None
    with torch.cuda.device(dout.device):
        rc = _lib.load().fsw_backward_dx_gate(
            dout.data_ptr(), g.data_ptr(), u.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), dx.data_ptr(),
            dg.data_ptr(), du.data_ptr(), T, dm, di, ws.data_ptr() if ws is not None else None,
            ws.numel() if ws is not None else 0, _code(dout), _stream(dout))
    _lib.check("fsw_backward_dx_gate", rc)
    return dx, dg, du


def gate_grad_from_factors(dout: torch.Tensor, s: torch.Tensor, t: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(dg, du) = (dout * t, dout * s) as a kernel of its own."""
    _require_cuda(dout, s, t)
    dg, du = torch.empty_like(dout), torch.empty_like(dout)
    with torch.cuda.device(dout.device):
        rc = _lib.load().fsw_backward_elementwise_st(
            dout.data_ptr(), s.data_ptr(), t.data_ptr(), dg.data_ptr(), du.data_ptr(), dout.numel(),
            _code(dout), _stream(dout))
    _lib.check("fsw_backward_elementwise_st", rc)
    return dg, du


def _ptr_array(ptrs):
    import ctypes

    return (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def grad_input_scatter(dg: torch.Tensor, du: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                       recv_ptrs, world: int, rank: int) -> None:
    """The dX GEMM of one rank of a column-parallel group; its epilogue stores the
    partial sums into the owning ranks' receive buffers (``recv_ptrs``: one device
    pointer per rank, peer memory mapped into this process; see fsw_backward_dx_scatter)."""
    _require_cuda(dg, du, w_gate, w_up)
    T, di = dg.shape
    dm = w_gate.shape[0]
    with torch.cuda.device(dg.device):
        rc = _lib.load().fsw_backward_dx_scatter(
            dg.data_ptr(), du.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), _ptr_array(recv_ptrs),
            int(world), int(rank), T, dm, di, _code(dg), _lib.FSW_ACC_F32, _stream(dg),
        )
    _lib.check("fsw_backward_dx_scatter", rc)


def reduce_dx_slices(recv_ptr: int, peer_flag_ptrs, my_flags_ptr: int, world: int, rank: int, seq: int,
                     out: torch.Tensor, own_slice: Optional[torch.Tensor] = None) -> None:
    """Signal the peers, wait (bounded) for their partials and sum the ``world`` slices
    of this rank's receive buffer into ``out`` (rows, dm); see fsw_dx_reduce."""
    rows, dm = out.shape
    with torch.cuda.device(out.device):
        rc = _lib.load().fsw_dx_reduce(
            recv_ptr, own_slice.data_ptr() if own_slice is not None else None, _ptr_array(peer_flag_ptrs), my_flags_ptr, int(world), int(rank), int(seq) & 0xFFFFFFFF,
            rows, dm, out.data_ptr(), _code(out), _stream(out),
        )
    _lib.check("fsw_dx_reduce", rc)


def wait_flags(flags_ptr: int, n: int, seq: int, like: torch.Tensor) -> None:
    """Queue a time-limited wait until ``n`` 32-bit flag words have reached ``seq``."""
    with torch.cuda.device(like.device):
        rc = _lib.load().fsw_wait_flags(flags_ptr, int(n), int(seq) & 0xFFFFFFFF, _stream(like))
    _lib.check("fsw_wait_flags", rc)

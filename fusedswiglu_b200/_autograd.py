"""Shared forward/backward of the two autograd Functions.

Mirrors the data flow of the reference's ``FusedSwiGLU`` (fused_swiglu/swiglu.py:16-58):
forward saves ``(x, w_gate, w_up, x@w_gate, x@w_up)`` and returns only ``out``;
backward runs the gate-gradient step, the input-gradient GEMM and the
weight-gradient GEMM and returns ``(dX, dW_gate, dW_up)``.

Differences, all on the accurate side of the reference's tolerances:
  * dX is ONE GEMM accumulating both products in fp32 (the reference rounds each
    product to 16 bits and adds, swiglu.py:45);
  * dW is reduced over all bs*sq tokens in one launch with a single rounding (the
    reference rounds per batch and sums in 16 bits, swiglu.py:51-57), and is
    returned as (d_model, d_intermediate) - autograd reduces the reference's
    (1, d_model, d_intermediate) to that shape anyway;
  * gradients that autograd does not need are not computed;
  * with ``recompute`` the saved x@w_gate and x@w_up are dropped and recomputed in
    backward (an activation-memory mode the reference does not have);
  * with ``fused_gate_grad`` the forward saves s = silu(g) and t = u*silu'(g) instead
    of g and u, and the gate-gradient step runs inside the dX GEMM (one launch for
    kernels_bf16.py:210-255 + swiglu.py:45): dg = dout*t, du = dout*s, one rounding
    apart from the reference's order (dout*u first, then *silu'(g)).
"""
from __future__ import annotations

import torch

from . import _launch


def swiglu_forward(ctx, x, w_gate, w_up, *, fast_accum: bool, recompute: bool = False,
                   fused_gate_grad: bool = False):
    assert (
        x.shape[2] == w_up.shape[0]
    ), f"Dimension mismatch. Expected a.shape[2] ({x.shape[2]}) to be equal to b.shape[0] ({w_up.shape[0]})"
    assert w_up.shape == w_gate.shape, "Expected both weight matrices to have same shape"
    assert x.ndim == 3 and w_up.ndim == 2, "Incorrect number of dimensions for LHS or RHS"
    assert x.dtype == w_gate.dtype == w_up.dtype, "Expected input and weights of one dtype"
    bs, sq, dm = x.shape
    di = w_up.shape[1]
    x2d = x.contiguous().view(bs * sq, dm)
    wg = w_gate.contiguous()
    wu = w_up.contiguous()
    # Grad mode is always off inside Function.forward; what autograd will ask for
    # is in ctx.needs_input_grad (all False under torch.no_grad()).
    need_grad = any(ctx.needs_input_grad[:3])
    # recompute: keep only x and the weights; backward runs the forward kernel again to
    # get g and u (bit-identical), trading one extra dual GEMM for 2*T*di saved elements.
    save_gu = need_grad and not recompute
    ctx.fused_gate_grad = bool(fused_gate_grad)
    out, g, u = _launch.forward(x2d, wg, wu, fast_accum=fast_accum, save_activations=save_gu,
                                save_factors=save_gu and ctx.fused_gate_grad)
    if save_gu:
        ctx.save_for_backward(x2d, wg, wu, g, u)
    elif need_grad:
        ctx.save_for_backward(x2d, wg, wu)
    ctx.in_shape = (bs, sq, dm)
    return out.view(bs, sq, di)


def swiglu_backward(ctx, grad_output, *, fast_accum: bool):
    if len(ctx.saved_tensors) == 5:
        x2d, wg, wu, g, u = ctx.saved_tensors
    else:
        x2d, wg, wu = ctx.saved_tensors
        _, g, u = _launch.forward(x2d, wg, wu, fast_accum=fast_accum, save_activations=True,
                                  save_factors=ctx.fused_gate_grad)
    bs, sq, dm = ctx.in_shape
    di = wg.shape[1]
    need_x, need_g, need_u = ctx.needs_input_grad[:3]
    dout = grad_output.contiguous().view(bs * sq, di)
    if dout.dtype != x2d.dtype:
        dout = dout.to(x2d.dtype)
    dx = dwg = dwu = None
    if ctx.fused_gate_grad:  # g and u hold the saved factors s and t
        if need_x:
            dx, dg, du = _launch.grad_input_fused(dout, g, u, wg, wu)
            dx = dx.view(bs, sq, dm)
        else:
            dg, du = _launch.gate_grad_from_factors(dout, g, u)
    else:
        dg, du = _launch.gate_grad(dout, g, u)
        if need_x:
            dx = _launch.grad_input(dg, du, wg, wu).view(bs, sq, dm)
    if need_g or need_u:
        dwg, dwu = _launch.grad_weights(x2d, dg, du, fast_accum=fast_accum)
        dwg = dwg if need_g else None
        dwu = dwu if need_u else None
    return dx, dwg, dwu

"""Module-level launchers with the names and return orders of the reference's
``fused_swiglu/kernels/kernels_bf16.py`` and ``kernels_fp16.py``; the two public
modules differ only in the dtype they accept and the accumulate default."""
from __future__ import annotations

from typing import Tuple

import torch

from .. import _launch


def check_fwd_args(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor) -> None:
    # Same assertions, in the same order, as fused_swiglu_fwd in the reference
    # (kernels_bf16.py:170-180).
    assert (
        x.shape[2] == w_up.shape[0]
    ), f"Dimension mismatch. Expected a.shape[2] ({x.shape[2]}) to be equal to b.shape[0] ({w_up.shape[0]})"
    assert w_up.shape == w_gate.shape, "Expected both weight matrices to have same shape"
    assert x.ndim == 3 and w_up.ndim == 2, "Incorrect number of dimensions for LHS or RHS"


def fwd(x, w_gate, w_up, fast_accum: bool, save_activations: bool = True):
    B, M, N = x.shape
    K = w_up.shape[1]
    out, g, u = _launch.forward(
        x.contiguous().view(B * M, N), w_gate.contiguous(), w_up.contiguous(),
        fast_accum=fast_accum, save_activations=save_activations,
    )
    shape = (B, M, K)
    return out.view(shape), (g.view(shape) if g is not None else None), (u.view(shape) if u is not None else None)


def elementwise_backward(
    grad_output: torch.Tensor, xw_gate: torch.Tensor, xw_up: torch.Tensor
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gate-gradient step.  Returns ``(grad_xw_up, grad_xw_gate)`` - up first, as
    the reference does (kernels_bf16.py:236-255)."""
    assert grad_output.shape == xw_gate.shape == xw_up.shape, "Expected equal shapes"
    dg, du = _launch.gate_grad(grad_output.contiguous(), xw_gate.contiguous(), xw_up.contiguous())
    return du, dg


def fused_bmm(
    x: torch.Tensor, grad_xw_up: torch.Tensor, grad_xw_gate: torch.Tensor, fast_accum: bool
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-batch weight gradients, ``(grad_weight_up, grad_weight_gate)`` of shape
    (B, d_model, d_intermediate), for ``x`` given as (B, d_model, sq) - the layout
    the reference passes (kernels_bf16.py:385-412, swiglu.py:51).

    The autograd Functions do not use this: they reduce over every token in one
    launch.  It exists for callers of the reference's module-level function."""
    assert (
        x.shape[-1] == grad_xw_up.shape[-2]
    ), f"Dimension mismatch. Expected a.shape[2] ({x.shape[-1]}) to be equal to b.shape[0] ({grad_xw_up.shape[-2]})"
    assert x.ndim == 3 and grad_xw_up.ndim == 3, "Incorrect number of dimensions for LHS or RHS"
    B, M, _ = x.shape
    K = grad_xw_up.shape[2]
    x_rows = x.transpose(1, 2).contiguous()  # (B, sq, d_model)
    du = grad_xw_up.contiguous()
    dg = grad_xw_gate.contiguous()
    gw_up = torch.empty((B, M, K), device=x.device, dtype=x.dtype)
    gw_gate = torch.empty((B, M, K), device=x.device, dtype=x.dtype)
    for b in range(B):
        _launch.grad_weights(x_rows[b], dg[b], du[b], fast_accum=fast_accum,
                             out_gate=gw_gate[b], out_up=gw_up[b])
    return gw_up, gw_gate

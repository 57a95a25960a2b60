"""SwiGLU MLP block: ``y = (silu(x @ w_gate) * (x @ w_up)) @ w_down``.

The reference stops at the SwiGLU output; every Llama-style MLP multiplies it by a
down projection next.  ``FusedSwiGLUMLP`` runs that projection and its two gradients
on the same tcgen05 GEMM kernel (``fsw_gemm``), so the whole block - five GEMM
launches and one elementwise launch per forward+backward - stays in this library.

Shapes: x (bs, sq, d_model); w_gate, w_up (d_model, d_intermediate);
w_down (d_intermediate, d_out); y (bs, sq, d_out).
"""
from __future__ import annotations

import math

import torch
from torch import nn
from torch.autograd import Function

from . import _launch


class FusedSwiGLUMLP(Function):
    """``FusedSwiGLUMLP.apply(x, w_gate, w_up, w_down)`` for bf16 (fp32 accumulation)
    or fp16 tensors (fp32 accumulation; the fp16 accumulator is a FastAccumFusedSwiGLU
    option and is not used here)."""

    @staticmethod
    def forward(ctx, x, w_gate, w_up, w_down):
        assert x.ndim == 3 and w_gate.ndim == 2 and w_down.ndim == 2, "Incorrect number of dimensions"
        assert w_gate.shape == w_up.shape, "Expected both weight matrices to have same shape"
        assert x.shape[2] == w_gate.shape[0] and w_gate.shape[1] == w_down.shape[0], "Dimension mismatch"
        assert x.dtype == w_gate.dtype == w_up.dtype == w_down.dtype, "Expected tensors of one dtype"
        bs, sq, dm = x.shape
        x2d = x.contiguous().view(bs * sq, dm)
        wg, wu, wd = w_gate.contiguous(), w_up.contiguous(), w_down.contiguous()
        need = any(ctx.needs_input_grad)
        out, g, u = _launch.forward(x2d, wg, wu, save_activations=need)
        y = _launch.gemm(out, wd)
        if need:
            ctx.save_for_backward(x2d, wg, wu, wd, g, u, out)
        ctx.in_shape = (bs, sq, dm)
        return y.view(bs, sq, wd.shape[1])

    @staticmethod
    def backward(ctx, grad_y):
        x2d, wg, wu, wd, g, u, out = ctx.saved_tensors
        bs, sq, dm = ctx.in_shape
        need_x, need_g, need_u, need_d = ctx.needs_input_grad
        dy = grad_y.contiguous().view(bs * sq, wd.shape[1])
        dwd = _launch.gemm(out, dy, trans_a=True) if need_d else None     # out^T @ dy
        dx = dwg = dwu = None
        if need_x or need_g or need_u:
            dout = _launch.gemm(dy, wd, trans_b=True)                      # dy @ w_down^T
            dg, du = _launch.gate_grad(dout, g, u)
            if need_x:
                dx = _launch.grad_input(dg, du, wg, wu).view(bs, sq, dm)
            if need_g or need_u:
                dwg, dwu = _launch.grad_weights(x2d, dg, du)
                dwg = dwg if need_g else None
                dwu = dwu if need_u else None
        return dx, dwg, dwu, dwd


class SwiGLUMLP(nn.Module):
    """Llama-style MLP block with parameters in (in_features, out_features) layout."""

    def __init__(self, d_model: int, d_intermediate: int, d_out: int | None = None,
                 dtype: torch.dtype = torch.bfloat16, device=None):
        super().__init__()
        d_out = d_model if d_out is None else d_out
        if dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("SwiGLUMLP supports torch.bfloat16 and torch.float16 parameters")
        if d_model % 8 or d_intermediate % 8 or d_out % 8:
            raise ValueError("feature sizes must be multiples of 8")

        def init(rows, cols):
            w = torch.randn(rows, cols, device=device, dtype=torch.float32).mul_(1.0 / math.sqrt(rows))
            return nn.Parameter(w.to(dtype))

        self.w_gate, self.w_up = init(d_model, d_intermediate), init(d_model, d_intermediate)
        self.w_down = init(d_intermediate, d_out)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return FusedSwiGLUMLP.apply(x, self.w_gate, self.w_up, self.w_down)

"""``FusedSwiGLU``: bf16 SwiGLU with fp32 accumulation on B200 tensor cores.

Drop-in for the reference's ``fused_swiglu.swiglu.FusedSwiGLU``
(fused_swiglu/swiglu.py:16-58): ``FusedSwiGLU.apply(x, w_gate, w_up)`` with
x (bs, sq, d_model) and weights (d_model, d_intermediate)."""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import _autograd


class FusedSwiGLU(Function):
    # Set to True to save only x and the weights and recompute x@w_gate, x@w_up in
    # backward: frees 2*bs*sq*d_intermediate saved elements for one more dual GEMM.
    recompute_activations = False
    # Set to True to run the gate-gradient step inside the dX GEMM: the forward then saves
    # silu(g) and u*silu'(g) instead of g and u, and backward launches two kernels, not three.
    fused_gate_grad = False

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, input: torch.Tensor, weight_gate: torch.Tensor, weight_up: torch.Tensor) -> torch.Tensor:
        assert input.dtype == torch.bfloat16, "Expected torch.bfloat16 inputs and weights."
        return _autograd.swiglu_forward(ctx, input, weight_gate, weight_up, fast_accum=False,
                                        recompute=bool(FusedSwiGLU.recompute_activations),
                                        fused_gate_grad=bool(FusedSwiGLU.fused_gate_grad))

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        return _autograd.swiglu_backward(ctx, grad_output, fast_accum=False)

"""``FastAccumFusedSwiGLU``: fp16 SwiGLU with an fp16 tensor-memory accumulator.

Drop-in for the reference's ``fused_swiglu.swiglu_f16.FastAccumFusedSwiGLU``
(fused_swiglu/swiglu_f16.py:16-58).  As there, ``.apply`` always uses fp16
accumulation in the forward GEMM and in the weight-gradient GEMM, and fp32
accumulation for the input gradient.  Set ``FastAccumFusedSwiGLU.fast_accum =
False`` to accumulate everything in fp32 (the reference reaches that only through
``fused_swiglu_fwd(..., fast_accum=False)``, kernels_fp16.py:172)."""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import _autograd


class FastAccumFusedSwiGLU(Function):
    fast_accum = True
    recompute_activations = False  # see FusedSwiGLU.recompute_activations
    fused_gate_grad = False        # see FusedSwiGLU.fused_gate_grad

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, input: torch.Tensor, weight_gate: torch.Tensor, weight_up: torch.Tensor) -> torch.Tensor:
        assert input.dtype == torch.float16, "Expected torch.float16 inputs and weights."
        ctx.fast_accum = bool(FastAccumFusedSwiGLU.fast_accum)
        return _autograd.swiglu_forward(ctx, input, weight_gate, weight_up, fast_accum=ctx.fast_accum,
                                        recompute=bool(FastAccumFusedSwiGLU.recompute_activations),
                                        fused_gate_grad=bool(FastAccumFusedSwiGLU.fused_gate_grad))

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        return _autograd.swiglu_backward(ctx, grad_output, fast_accum=ctx.fast_accum)

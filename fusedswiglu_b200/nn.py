"""``torch.nn`` wrapper around the fused SwiGLU Functions.

The reference ships only the autograd Functions; this module is a convenience for
model code: it owns ``w_gate`` and ``w_up`` in the reference's layout
``(d_model, d_intermediate)`` and calls ``FusedSwiGLU`` (bf16) or
``FastAccumFusedSwiGLU`` (fp16) according to the parameter dtype.
"""
from __future__ import annotations

import math

import torch
from torch import nn

from .swiglu import FusedSwiGLU
from .swiglu_f16 import FastAccumFusedSwiGLU


class SwiGLU(nn.Module):
    """``out = silu(x @ w_gate) * (x @ w_up)`` for x of shape (bs, sq, d_model)."""

    def __init__(self, d_model: int, d_intermediate: int, dtype: torch.dtype = torch.bfloat16, device=None):
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("SwiGLU supports torch.bfloat16 and torch.float16 parameters")
        if d_model % 8 or d_intermediate % 8:
            raise ValueError("d_model and d_intermediate must be multiples of 8")
        self.d_model, self.d_intermediate = d_model, d_intermediate
        scale = 1.0 / math.sqrt(d_model)
        self.w_gate = nn.Parameter(torch.randn(d_model, d_intermediate, device=device, dtype=torch.float32).mul_(scale).to(dtype))
        self.w_up = nn.Parameter(torch.randn(d_model, d_intermediate, device=device, dtype=torch.float32).mul_(scale).to(dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        fn = FusedSwiGLU if self.w_gate.dtype == torch.bfloat16 else FastAccumFusedSwiGLU
        return fn.apply(x, self.w_gate, self.w_up)

    def extra_repr(self) -> str:
        return f"d_model={self.d_model}, d_intermediate={self.d_intermediate}, dtype={self.w_gate.dtype}"

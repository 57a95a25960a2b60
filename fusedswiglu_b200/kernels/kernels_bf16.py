"""bf16 launchers (fp32 accumulation), the counterpart of the reference's
``fused_swiglu/kernels/kernels_bf16.py`` host functions (:162-206, :236-255,
:385-412), backed by tcgen05 kernels instead of Triton."""
from __future__ import annotations

from typing import Tuple

import torch

from . import _common

elementwise_backward = _common.elementwise_backward


def fused_swiglu_fwd(
    x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(out, x@w_gate, x@w_up)`` for x (bs, sq, d_model), weights (d_model, d_intermediate)."""
    _common.check_fwd_args(x, w_gate, w_up)
    assert x.dtype == torch.bfloat16, "Expected torch.bfloat16 inputs and weights."
    return _common.fwd(x, w_gate, w_up, fast_accum=False)


def fused_bmm(x, grad_xw_up, grad_xw_gate):
    return _common.fused_bmm(x, grad_xw_up, grad_xw_gate, fast_accum=False)

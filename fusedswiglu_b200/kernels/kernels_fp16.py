"""fp16 launchers, the counterpart of the reference's
``fused_swiglu/kernels/kernels_fp16.py`` host functions (:171-216, :246-265,
:395-422).  ``fast_accum=True`` (the default there, :172) keeps the forward
accumulators in fp16 tensor memory; the per-batch weight-gradient GEMM always
accumulates in fp16 (:318-319)."""
from __future__ import annotations

from typing import Tuple

import torch

from . import _common

elementwise_backward = _common.elementwise_backward


def fused_swiglu_fwd(
    x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, fast_accum: bool = True
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    _common.check_fwd_args(x, w_gate, w_up)
    assert x.dtype == torch.float16, "Expected torch.float16 inputs and weights."
    return _common.fwd(x, w_gate, w_up, fast_accum=fast_accum)


def fused_bmm(x, grad_xw_up, grad_xw_gate):
    return _common.fused_bmm(x, grad_xw_up, grad_xw_gate, fast_accum=True)

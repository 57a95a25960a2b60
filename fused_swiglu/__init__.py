"""Import-name compatibility with fattorib/fusedswiglu: ``from fused_swiglu import
FusedSwiGLU, FastAccumFusedSwiGLU`` and the submodule paths ``fused_swiglu.swiglu``,
``fused_swiglu.swiglu_f16`` and ``fused_swiglu.kernels.kernels_{bf16,fp16}`` all
resolve to the B200 implementation in ``fusedswiglu_b200``."""
import sys

import fusedswiglu_b200
from fusedswiglu_b200 import FastAccumFusedSwiGLU, FusedSwiGLU, kernels, swiglu, swiglu_f16
from fusedswiglu_b200.kernels import kernels_bf16, kernels_fp16

for _name, _mod in {
    "swiglu": swiglu,
    "swiglu_f16": swiglu_f16,
    "kernels": kernels,
    "kernels.kernels_bf16": kernels_bf16,
    "kernels.kernels_fp16": kernels_fp16,
}.items():
    sys.modules[f"{__name__}.{_name}"] = _mod

__all__ = ["FusedSwiGLU", "FastAccumFusedSwiGLU"]

"""B200-native fused SwiGLU with the API of fattorib/fusedswiglu.

    from fusedswiglu_b200 import FusedSwiGLU, FastAccumFusedSwiGLU
    out = FusedSwiGLU.apply(x, w_gate, w_up)

``import fused_swiglu`` (the reference's package name) re-exports the same names.
All arithmetic runs in libfused_swiglu_sm100.so (sm_100a TMA + tcgen05 kernels);
there is no Triton, PyTorch or CPU fallback.
"""
from .swiglu import FusedSwiGLU
from .swiglu_f16 import FastAccumFusedSwiGLU

__all__ = ["FusedSwiGLU", "FastAccumFusedSwiGLU"]
__version__ = "0.1.0"

"""Host-side behaviour that needs no GPU: the reference's API surface and error
conventions, and the refusal to run anywhere but on CUDA tensors."""
import pytest
import torch


def test_reference_import_paths_resolve():
    import fused_swiglu
    from fused_swiglu import FastAccumFusedSwiGLU, FusedSwiGLU
    from fused_swiglu.kernels.kernels_bf16 import elementwise_backward, fused_bmm, fused_swiglu_fwd
    from fused_swiglu.kernels import kernels_fp16
    from fused_swiglu.swiglu import FusedSwiGLU as F2
    from fused_swiglu.swiglu_f16 import FastAccumFusedSwiGLU as H2

    assert F2 is FusedSwiGLU and H2 is FastAccumFusedSwiGLU
    assert issubclass(FusedSwiGLU, torch.autograd.Function)
    assert issubclass(FastAccumFusedSwiGLU, torch.autograd.Function)
    assert callable(elementwise_backward) and callable(fused_bmm) and callable(fused_swiglu_fwd)
    assert callable(kernels_fp16.fused_swiglu_fwd)
    assert fused_swiglu.__all__ == ["FusedSwiGLU", "FastAccumFusedSwiGLU"]


def _args(dm=64, di=128, dtype=torch.bfloat16):
    return (torch.zeros(1, 64, dm, dtype=dtype), torch.zeros(dm, di, dtype=dtype), torch.zeros(dm, di, dtype=dtype))


def test_shape_assertions_match_the_reference_messages():
    from fused_swiglu.kernels.kernels_bf16 import fused_swiglu_fwd

    x, wg, wu = _args()
    with pytest.raises(AssertionError, match="Dimension mismatch"):
        fused_swiglu_fwd(x, torch.zeros(32, 128, dtype=x.dtype), torch.zeros(32, 128, dtype=x.dtype))
    with pytest.raises(AssertionError, match="same shape"):
        fused_swiglu_fwd(x, torch.zeros(64, 64, dtype=x.dtype), wu)
    with pytest.raises(AssertionError, match="bfloat16"):
        fused_swiglu_fwd(x.half(), wg.half(), wu.half())
    with pytest.raises(AssertionError, match="Dimension mismatch"):
        from fused_swiglu import FusedSwiGLU

        FusedSwiGLU.apply(x, torch.zeros(32, 128, dtype=x.dtype), torch.zeros(32, 128, dtype=x.dtype))


def test_cpu_tensors_are_refused_loudly():
    from fused_swiglu import FastAccumFusedSwiGLU, FusedSwiGLU

    with pytest.raises(RuntimeError, match="no CPU path"):
        FusedSwiGLU.apply(*_args())
    with pytest.raises(RuntimeError, match="no CPU path"):
        FastAccumFusedSwiGLU.apply(*_args(dtype=torch.float16))


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    from fusedswiglu_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_product_does_not_import_the_oracle():
    import pathlib

    pkg = pathlib.Path(__file__).resolve().parent.parent / "fusedswiglu_b200"
    for p in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu")) + list(pkg.rglob("*.cuh")):
        text = p.read_text()
        for needle in ("import oracle", "from oracle", "swiglu_oracle", "oracle/", "oracle."):
            assert needle not in text, f"{p} refers to the oracle package ({needle!r})"

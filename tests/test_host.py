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


def test_bench_parity_report_on_cpu_tensors():
    """The bench's per-tensor parity reporter, fed from the CPU: exact float64 results give
    errors at the level of one bf16 rounding, a corrupted tensor is flagged above the bound."""
    import torch

    import bench

    torch.manual_seed(0)
    T, dm, di = 192, 64, 96
    x = torch.randn(T, dm).bfloat16()
    wg, wu = (torch.randn(dm, di) / dm ** 0.5).bfloat16(), (torch.randn(dm, di) / dm ** 0.5).bfloat16()
    dout = torch.randn(T, di).bfloat16()
    g, u = x.double() @ wg.double(), x.double() @ wu.double()
    s = torch.sigmoid(g)
    out = torch.nn.functional.silu(g) * u
    dg, du = dout.double() * u * (s + g * s * (1 - s)), dout.double() * g * s
    dx = dg @ wg.double().T + du @ wu.double().T
    dwg, dwu = x.double().T @ dg, x.double().T @ du
    good = [t.bfloat16() for t in (out, dx, dwg, dwu)]
    rep = bench.parity_report(x, wg, wu, dout, *good, world=1)
    assert rep["ok"] and all(rep[k]["rel_fro"] < 4e-3 for k in ("out", "dx", "dw_gate", "dw_up")), rep
    assert all(rep[k]["max_abs"] >= 0 and rep[k]["max_rel"] >= 0 for k in ("out", "dx", "dw_gate", "dw_up"))
    bad = list(good)
    bad[1] = (dx * 1.05).bfloat16()  # 5 % off: far above the 1e-2 bound
    rep = bench.parity_report(x, wg, wu, dout, *bad, world=1)
    assert not rep["ok"] and rep["dx"]["rel_fro"] > 1e-2 and rep["out"]["rel_fro"] < 4e-3


def test_bench_cpu_sample_rule_and_sampler_without_a_gpu():
    import time

    import bench

    # the whole 8B workload fits the CPU budget, the 70B one is cut to T/8
    assert bench.cpu_sample_tokens(32768, 4096, 14336) == 32768
    assert bench.cpu_sample_tokens(65536, 8192, 28672) == 8192
    assert bench.flops_per_step(32768, 4096, 14336) == 12.0 * 32768 * 4096 * 14336
    assert bench.host_threads() >= 1
    # without NVML / nvidia-smi the sampler yields an empty record instead of failing
    s = bench.ClockSampler("GPU-00000000-0000-0000-0000-000000000000", 0)
    t0 = time.time()
    s.start()
    rec = s.summary(t0, time.time() + 1, "test")
    assert rec["samples"] >= 0 and "reasons" in rec
    assert bench.load_dram_traffic("fwd_dual_gemm", "llama3_8b_mlp", 1) > 1e9
    assert bench.load_dram_traffic("fwd_dual_gemm", "llama3_8b_mlp", 8) is None

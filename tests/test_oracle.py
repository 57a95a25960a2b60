"""The CPU oracle against the golden vectors produced by the reference's own
``swiglu_ref_torch`` (tests/golden/make_golden.py), and its internal consistency."""
import numpy as np
import pytest

from conftest import GOLDEN_CASES, load_golden
from oracle import swiglu_oracle as orc

# The reference's own bound for bf16 (test_swiglu.py:20) - and what it "expects".
REF_TOL = 1e-2
EXPECTED = 2e-3


def test_bf16_rounding_matches_torch():
    import torch

    rng = np.random.default_rng(1)
    a = np.concatenate([
        rng.standard_normal(4096).astype(np.float32) * 100,
        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38, 1e-40, np.inf, -np.inf], np.float32),
    ])
    want = torch.from_numpy(a).to(torch.bfloat16).float().numpy()
    got = orc.round_bf16(a)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(orc.from_bits(orc.to_bits(got, "bf16"), "bf16").view(np.uint32), got.view(np.uint32))


def test_fp16_bits_roundtrip():
    a = orc.round_fp16(np.linspace(-70000, 70000, 1001, dtype=np.float32))
    assert np.array_equal(orc.from_bits(orc.to_bits(a, "fp16"), "fp16"), a)


def test_reference_shape_generator_first_cases():
    # First forward and backward cases the reference's seeded comprehensions yield
    # with numpy's legacy seed 0.
    fwd, bwd = orc.reference_test_shapes()
    assert len(fwd) == 81 and len(bwd) == 81
    assert fwd[0] == (1, 256, 6656, 1408)
    assert bwd[0] == (2, 1152, 2304, 4480)
    for lst in (fwd, bwd):
        for b, sq, dm, di in lst:
            assert 1 <= b <= 3 and sq % 64 == 0 and dm % 64 == 0 and di % 64 == 0


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_oracle_matches_reference_golden(name):
    c = load_golden(name)
    dt, step = c["dtype"], c["row_step"]
    out = orc.swiglu_ref(c["x"], c["w_gate"], c["w_up"], dt)
    dx, dwg, dwu = orc.swiglu_ref_backward(c["x"], c["w_gate"], c["w_up"], c["dout"], dt)
    got = {"out": out, "dx": dx, "dw_gate": dwg[::step], "dw_up": dwu[::step]}
    for k, v in got.items():
        rep = orc.error_report(v, c[k])
        # Same formula, same rounding points; only GEMM summation order differs,
        # which moves a few results by one 16-bit ulp.
        assert rep["rel_fro"] < 5e-4, (name, k, rep)
        mism = np.mean(orc.to_bits(v, dt) != orc.to_bits(c[k], dt))
        assert mism < 0.05, (name, k, mism)


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_kernel_order_restatement_within_reference_tolerance(name):
    c = load_golden(name)
    dt, step = c["dtype"], c["row_step"]
    out, g, u = orc.kernel_forward(c["x"], c["w_gate"], c["w_up"], dt)
    dx, dwg, dwu = orc.kernel_backward(c["x"], c["w_gate"], c["w_up"], g, u, c["dout"], dt)
    got = {"out": out, "dx": dx, "dw_gate": dwg[::step], "dw_up": dwu[::step]}
    for k, v in got.items():
        e = orc.rel_error(v, c[k])
        assert e < REF_TOL, (name, k, e)
        assert e < (EXPECTED if dt == "fp16" else 3 * EXPECTED), (name, k, e)


def test_elementwise_backward_order_and_formula():
    rng = np.random.default_rng(3)
    g = orc.round_bf16(rng.standard_normal(1000).astype(np.float32) * 3)
    u = orc.round_bf16(rng.standard_normal(1000).astype(np.float32))
    d = orc.round_bf16(rng.standard_normal(1000).astype(np.float32))
    du, dg = orc.kernel_elementwise_backward(d, g, u, "bf16")
    g64 = g.astype(np.float64)
    s = 1 / (1 + np.exp(-g64))
    assert orc.rel_error(du, d * g64 * s) < 5e-3
    assert orc.rel_error(dg, d * u * (s + g64 * s * (1 - s))) < 5e-3


def test_silu_extremes_are_finite():
    g = np.array([-200.0, -90.0, -20.0, 0.0, 20.0, 90.0, 200.0], np.float32)
    assert np.all(np.isfinite(orc.silu_f32(g))) and np.all(np.isfinite(orc.silu_grad_f32(g)))
    assert orc.silu_f32(g)[0] == 0 and orc.silu_f32(g)[-1] == 200.0
    assert orc.silu_grad_f32(g)[-1] == 1.0


def test_torch_form_matches_numpy_form():
    import torch

    inp = orc.make_inputs(2, 64, 128, 192, "bf16", seed=5)
    t = {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in inp.items()}
    out_t = orc.swiglu_ref_torch(t["x"], t["w_gate"], t["w_up"]).float().numpy()
    out_n = orc.swiglu_ref(inp["x"], inp["w_gate"], inp["w_up"], "bf16")
    assert orc.rel_error(out_t, out_n) < 5e-4


def test_empty_input():
    x = np.zeros((1, 0, 64), np.float32)
    w = np.ones((64, 128), np.float32)
    assert orc.swiglu_ref(x, w, w).shape == (1, 0, 128)

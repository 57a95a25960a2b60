"""Parity of the CUDA path (called through the C ABI) with the CPU oracle, the
golden vectors of the reference's own PyTorch SwiGLU, and the reference's own
test recipe.  Everything here needs a B200."""
import math
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_CASES, load_golden
from oracle import swiglu_oracle as orc

pytestmark = pytest.mark.gpu

# The reference's bound on ||a-b||_F/||b||_F for out, dX, dW_gate, dW_up
# (fused_swiglu/test_swiglu.py:20) and the level it says to expect.
BFLOAT16_MAX_TOL = 1e-2
EXPECTED_BF16 = 6e-3
EXPECTED_FP16 = 1e-3

TDT = {"bf16": torch.bfloat16, "fp16": torch.float16}


@pytest.fixture(scope="module", autouse=True)
def cuda_ready():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from fusedswiglu_b200 import _lib

    _lib.load()
    yield
    assert _lib.device_status() == 0, "a kernel gave up on a bounded wait"


def dev(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).to(TDT[dtype]).cuda()


def host(t):
    return t.detach().float().cpu().numpy()


def run_cuda(inp, dtype, fast_accum=False):
    """Forward + backward through the package's launchers (ctypes -> C ABI)."""
    from fusedswiglu_b200 import _launch

    bs, sq, dm = inp["x"].shape
    di = inp["w_gate"].shape[1]
    x = dev(inp["x"].reshape(bs * sq, dm), dtype)
    wg, wu = dev(inp["w_gate"], dtype), dev(inp["w_up"], dtype)
    dout = dev(inp["dout"].reshape(bs * sq, di), dtype)
    out, g, u = _launch.forward(x, wg, wu, fast_accum=fast_accum)
    dg, du = _launch.gate_grad(dout, g, u)
    dx = _launch.grad_input(dg, du, wg, wu)
    dwg, dwu = _launch.grad_weights(x, dg, du, fast_accum=fast_accum)
    torch.cuda.synchronize()
    return {
        "out": host(out).reshape(bs, sq, di), "g": host(g).reshape(bs, sq, di), "u": host(u).reshape(bs, sq, di),
        "dg": host(dg).reshape(bs, sq, di), "du": host(du).reshape(bs, sq, di),
        "dx": host(dx).reshape(bs, sq, dm), "dw_gate": host(dwg), "dw_up": host(dwu),
    }


# --------------------------------------------------------- golden fixtures --
@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_against_reference_golden(name, cta_group):
    from fusedswiglu_b200 import _lib

    c = load_golden(name)
    old = _lib.get_option("cta_group")
    _lib.set_option("cta_group", cta_group)
    try:
        got = run_cuda(c, c["dtype"])
    finally:
        _lib.set_option("cta_group", old)
    step = c["row_step"]
    got["dw_gate"], got["dw_up"] = got["dw_gate"][::step], got["dw_up"][::step]
    expected = EXPECTED_BF16 if c["dtype"] == "bf16" else EXPECTED_FP16
    for k in ("out", "dx", "dw_gate", "dw_up"):
        rep = orc.error_report(got[k], c[k])
        print(name, cta_group, k, rep)
        assert rep["rel_fro"] < BFLOAT16_MAX_TOL, (name, k, rep)
        assert rep["rel_fro"] < expected, (name, k, rep)


# ------------------------------------------ oracle, kernel rounding order --
RAGGED = [64, 128, 192, 320]


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("T", RAGGED)
def test_ragged_shapes_against_kernel_order_oracle(T, dtype):
    worst = {}
    for dm in RAGGED:
        for di in RAGGED:
            inp = orc.make_inputs(1, T, dm, di, dtype, seed=T + dm + di, dout_std=0.5)
            got = run_cuda(inp, dtype)
            _, g, u = orc.kernel_forward(inp["x"], inp["w_gate"], inp["w_up"], dtype)
            # out and the elementwise step are checked on the GPU's own g, u so that
            # one-ulp differences in g do not blur them; the forward rounds like the
            # reference's PyTorch oracle: round(round(silu(g16)) * u16)
            out = orc.swiglu_from_saved(got["g"], got["u"], dtype)
            du, dg = orc.kernel_elementwise_backward(inp["dout"], got["g"], got["u"], dtype)
            dx64 = got["dg"].reshape(T, di).astype(np.float64) @ inp["w_gate"].T.astype(np.float64) + \
                got["du"].reshape(T, di).astype(np.float64) @ inp["w_up"].T.astype(np.float64)
            dwg64 = inp["x"].reshape(T, dm).T.astype(np.float64) @ got["dg"].reshape(T, di).astype(np.float64)
            dwu64 = inp["x"].reshape(T, dm).T.astype(np.float64) @ got["du"].reshape(T, di).astype(np.float64)
            want = {"out": out, "g": g, "u": u, "dg": dg, "du": du,
                    "dx": orc.round16(dx64.astype(np.float32), dtype).reshape(1, T, dm),
                    "dw_gate": orc.round16(dwg64.astype(np.float32), dtype),
                    "dw_up": orc.round16(dwu64.astype(np.float32), dtype)}
            for k, w in want.items():
                e = orc.rel_error(got[k], w)
                worst[k] = max(worst.get(k, 0.0), e)
                # same rounding points as the oracle: only ulp-level flips remain
                assert e < 1e-3, (T, dm, di, k, e)
                mism = np.mean(orc.to_bits(got[k], dtype) != orc.to_bits(w, dtype))
                assert mism < 0.03, (T, dm, di, k, mism)
    print("worst rel error per tensor:", worst)


def test_gemm_outputs_are_bit_exact_against_wide_accumulation():
    """g, u, dX, dW are pure GEMMs with fp32 accumulation and one rounding: except
    for sums that land within an fp32 rounding of a bf16 tie, the bits must equal a
    float64-accumulated result."""
    inp = orc.make_inputs(2, 128, 256, 384, "bf16", seed=11, dout_std=0.5)
    got = run_cuda(inp, "bf16")
    _, g, u = orc.kernel_forward(inp["x"], inp["w_gate"], inp["w_up"], "bf16")
    for k, w in (("g", g), ("u", u)):
        mism = np.mean(orc.to_bits(got[k], "bf16") != orc.to_bits(w, "bf16"))
        assert mism < 2e-3, (k, mism)


# ----------------------------------------------- the reference's own tests --
def _ref_shapes():
    num = int(os.environ.get("NUM_TEST", "3"))
    return orc.reference_test_shapes(num)


def make_input_weights(bs, sq, d_model, d_intermediate, dtype=torch.bfloat16):
    # test_swiglu.py:23-40: randn in the 16-bit dtype, weights divided by sqrt(d_model)
    x = torch.randn((bs, sq, d_model), device="cuda:0", dtype=dtype).requires_grad_(True)
    w_gate = torch.randn((d_model, d_intermediate), device="cuda:0", dtype=dtype) / math.sqrt(d_model)
    w_up = torch.randn((d_model, d_intermediate), device="cuda:0", dtype=dtype) / math.sqrt(d_model)
    return x, w_gate.requires_grad_(True), w_up.requires_grad_(True)


def rel_error(x, y):
    return (torch.linalg.norm(x.float() - y.float()) / torch.linalg.norm(y.float())).item()


def test_reference_forward_suite():
    """test_swiglu_fwd (test_swiglu.py:58-78) over its 81 seeded shapes."""
    from fused_swiglu import FusedSwiGLU

    torch.manual_seed(0)
    worst = 0.0
    for dims in _ref_shapes()[0]:
        x, wg, wu = make_input_weights(*dims)
        with torch.no_grad():
            ref = orc.swiglu_ref_torch(x, wg, wu)
            out = FusedSwiGLU.apply(x, wg, wu)
        e = rel_error(out, ref)
        worst = max(worst, e)
        assert e < BFLOAT16_MAX_TOL, (dims, e)
    print("worst forward rel error over the reference's shapes:", worst)
    assert worst < EXPECTED_BF16


def test_reference_backward_suite():
    """test_swiglu_bwd (test_swiglu.py:81-114) over its 81 seeded shapes."""
    from fused_swiglu import FusedSwiGLU

    torch.manual_seed(0)
    worst = {}
    for dims in _ref_shapes()[1]:
        x, wg, wu = make_input_weights(*dims)
        ref = orc.swiglu_ref_torch(x, wg, wu)
        dy = 0.1 * torch.randn_like(ref)
        ref.backward(dy, retain_graph=True)
        want = [t.grad.clone() for t in (x, wg, wu)]
        x.grad, wg.grad, wu.grad = None, None, None
        out = FusedSwiGLU.apply(x, wg, wu)
        out.backward(dy, retain_graph=True)
        got = [t.grad.clone() for t in (x, wg, wu)]
        for name, a, b in zip(("dx", "dw_gate", "dw_up"), got, want):
            assert a.shape == b.shape
            e = rel_error(a, b)
            worst[name] = max(worst.get(name, 0.0), e)
            assert e < BFLOAT16_MAX_TOL, (dims, name, e)
    print("worst backward rel errors over the reference's shapes:", worst)
    assert max(worst.values()) < EXPECTED_BF16


@pytest.mark.parametrize("opts", [
    {"cta_group": 1, "nsub": 1}, {"cta_group": 2, "nsub": 1}, {"cta_group": 2, "nsub": 2},
    {"gemm_max_sms": 100}, {"gemm_max_sms": 3}, {"group_m": 1}, {"group_m": 5}, {"group_m": 24}, {"l2_a": 0}, {"l2_b": 0}, {"l2_out": 0},
])
def test_tile_and_scheduling_options_do_not_change_results(opts):
    """Every tile shape / rasterisation / SM-cap setting computes the same GEMMs, so
    the results must be bit-identical to the default configuration."""
    from fusedswiglu_b200 import _lib

    inp = orc.make_inputs(1, 1344, 448, 1216, "bf16", seed=21, dout_std=0.5)
    old = {k: _lib.get_option(k) for k in list(opts) + ["split_k"]}
    try:
        _lib.set_option("split_k", 0)  # a split along K adds in another order; it has its own test
        base = run_cuda(inp, "bf16")
        for k, v in opts.items():
            _lib.set_option(k, v)
        got = run_cuda(inp, "bf16")
    finally:
        for k, v in old.items():
            _lib.set_option(k, v)
    for k in base:
        assert np.array_equal(got[k], base[k]), (opts, k)


@pytest.mark.parametrize("opts", [
    {"pace_kb": 1}, {"pace_kb": 5}, {"pace_kb": 32, "pace_limit_us": 1},
    {"pace_kb": 3, "cta_group": 2, "nsub": 2}, {"pace_kb": 2, "cta_group": 2, "nsub": 1},
    {"pace_kb": 7, "gemm_max_sms": 50},
])
def test_producer_pacing_does_not_change_results(opts):
    """The producers' meeting points are advisory: with any spacing, with waits that
    run out at once (1 us limit) and on several waves of tiles with a ragged last
    wave, results are bit-identical to the free-running kernel and no error is
    recorded."""
    from fusedswiglu_b200 import _lib

    inp = orc.make_inputs(1, 4224, 512, 2304, "bf16", seed=33, dout_std=0.5)
    names = sorted(set(opts) | {"pace_kb", "split_k"})
    old = {k: _lib.get_option(k) for k in names}
    try:
        _lib.set_option("split_k", 0)
        _lib.set_option("pace_kb", 0)
        base = run_cuda(inp, "bf16")
        for k, v in opts.items():
            _lib.set_option(k, v)
        got = run_cuda(inp, "bf16")
        assert _lib.device_status() == 0
        if "pace_limit_us" not in opts:
            # every CTA was resident and on time: pacing was not switched off
            assert _lib.get_option("pace_off") == 0
    finally:
        for k, v in old.items():
            _lib.set_option(k, v)
    for k in base:
        assert np.array_equal(got[k], base[k]), (opts, k)


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
def test_weight_gradient_column_ranges_equal_the_full_gemm(dtype):
    """fsw_backward_dw_columns writes exactly the values of fsw_backward_dw into the
    named columns and nothing anywhere else, for ragged ranges too."""
    from fusedswiglu_b200 import _launch

    T, dm, di = 1000, 320, 1096
    inp = orc.make_inputs(1, T, dm, di, dtype, seed=5, dout_std=0.5)
    x = dev(inp["x"].reshape(T, dm), dtype)
    dg = dev(inp["dout"].reshape(T, di), dtype)
    du = dev((inp["dout"] * 0.5 + 0.25).reshape(T, di), dtype)
    full_g, full_u = _launch.grad_weights(x, dg, du)
    for first, count in [(0, 256), (256, 840), (8, 16), (1088, 8), (0, di), (512, 0)]:
        out_g = torch.full_like(full_g, 7.0)
        out_u = torch.full_like(full_u, -3.0)
        _launch.grad_weights(x, dg, du, out_gate=out_g, out_up=out_u, columns=(first, count))
        torch.cuda.synchronize()
        sl = slice(first, first + count)
        assert torch.equal(out_g[:, sl], full_g[:, sl]) and torch.equal(out_u[:, sl], full_u[:, sl])
        keep = torch.ones(di, dtype=torch.bool, device=out_g.device)
        keep[sl] = False
        assert bool((out_g[:, keep] == 7.0).all()) and bool((out_u[:, keep] == -3.0).all())


@pytest.mark.parametrize("dtype,fast", [("bf16", False), ("fp16", False), ("fp16", True)])
@pytest.mark.parametrize("T,dm,di", [
    (16384, 1024, 2560),   # dW: 4 x 10 = 40 tiles on 74 pairs, every pair gets about half a tile
    (6000, 2048, 4800),    # dW: 8 x 19 = 152 tiles = two whole waves + 4 tiles split 18 ways; dX: 96 tiles
                           # = one wave + 22 split; ragged T and di
    (8192, 512, 7176),     # dX: 32 x 1 tiles, K = 2 x 113 blocks; di is not a multiple of 64
])
def test_split_of_the_last_wave_along_k(T, dm, di, dtype, fast):
    """With a workspace the last partial wave of tiles is divided along K over all SM
    pairs and summed in a second kernel.  Same products, another association of the
    fp32 sums: the results must agree with the unsplit launch to within a rounding of
    the output type, and with float64 as closely as the unsplit launch does.  Run
    twice: the split is deterministic."""
    from fusedswiglu_b200 import _launch, _lib

    inp = orc.make_inputs(1, T, dm, di, dtype, seed=T + di, dout_std=0.5)
    x = dev(inp["x"].reshape(T, dm), dtype)
    wg, wu = dev(inp["w_gate"], dtype), dev(inp["w_up"], dtype)
    dg = dev(inp["dout"].reshape(T, di), dtype)
    du = dev((inp["dout"] * 0.5 + 0.125).reshape(T, di), dtype)
    plain = {"dx": _launch.grad_input(dg, du, wg, wu, split_k=False)}
    plain["dwg"], plain["dwu"] = _launch.grad_weights(x, dg, du, fast_accum=fast, split_k=False)
    got = []
    for _ in range(2):
        r = {"dx": _launch.grad_input(dg, du, wg, wu)}
        r["dwg"], r["dwu"] = _launch.grad_weights(x, dg, du, fast_accum=fast)
        got.append(r)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    ref = {"dx": dg.double() @ wg.double().T + du.double() @ wu.double().T,
           "dwg": x.double().T @ dg.double(), "dwu": x.double().T @ du.double()}
    changed = 0
    for k in plain:
        assert torch.equal(got[0][k], got[1][k]), k
        changed += int((got[0][k] != plain[k]).sum())
        e_split, e_plain = rel_error(got[0][k], ref[k]), rel_error(plain[k], ref[k])
        print(f"split-K {dtype} fast={fast} T={T} {k}: vs float64 {e_split:.3e} (unsplit {e_plain:.3e}), "
              f"vs unsplit {rel_error(got[0][k], plain[k]):.3e}")
        assert e_split < max(1.2 * e_plain, 1e-4), (k, e_split, e_plain)
        assert rel_error(got[0][k], plain[k]) < (8e-3 if fast else 2e-3), k
    # the split did run (some last bits differ) unless every partial sum happened to round alike
    assert changed > 0 or dtype == "fp16"


@pytest.mark.parametrize("dtype,fast,save", [("bf16", False, True), ("bf16", False, False), ("fp16", True, True)])
def test_split_of_the_forward_s_last_wave_along_k(dtype, fast, save):
    """The forward with a workspace: 8 x 11 = 88 tiles are one wave of 74 plus 14 tiles
    whose K loops (128 blocks) are divided over all SM pairs; the second kernel adds
    the pieces, rounds g and u and applies the SwiGLU epilogue.  Ragged T and di."""
    from fusedswiglu_b200 import _launch, _lib

    T, dm, di = 2000, 8192, 2808
    inp = orc.make_inputs(1, T, dm, di, dtype, seed=77)
    x, wg, wu = dev(inp["x"].reshape(T, dm), dtype), dev(inp["w_gate"], dtype), dev(inp["w_up"], dtype)
    plain = _launch.forward(x, wg, wu, fast_accum=fast, save_activations=save, split_k=False)
    a = _launch.forward(x, wg, wu, fast_accum=fast, save_activations=save)
    b = _launch.forward(x, wg, wu, fast_accum=fast, save_activations=save)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    g64, u64 = x.double() @ wg.double(), x.double() @ wu.double()
    ref = (torch.nn.functional.silu(g64) * u64, g64, u64)
    changed = 0
    for k, name in enumerate(("out", "g", "u")):
        if a[k] is None:
            assert not save and plain[k] is None
            continue
        assert torch.equal(a[k], b[k]), name
        changed += int((a[k] != plain[k]).sum())
        e_split, e_plain = rel_error(a[k], ref[k]), rel_error(plain[k], ref[k])
        print(f"forward split-K {dtype} fast={fast} {name}: vs float64 {e_split:.3e} (unsplit {e_plain:.3e})")
        assert e_split < max(1.2 * e_plain, 1e-4), (name, e_split, e_plain)
        assert rel_error(a[k], plain[k]) < (8e-3 if fast else 2e-3), name
    assert changed > 0 or dtype == "fp16"
    if save:
        # out is the epilogue applied to the g and u that were written (the GPU's fast
        # sigmoid may flip a last bit here and there)
        want = orc.swiglu_from_saved(host(a[1]), host(a[2]), dtype)
        assert np.mean(orc.to_bits(host(a[0]), dtype) != orc.to_bits(want, dtype)) < 0.01


def test_dw_beside_a_collective_in_two_parts_equals_one_launch(monkeypatch):
    """The split the column-parallel backward uses when the dW GEMM outlasts the
    all-reduce: first columns on fewer SMs, wait for the collective, rest on all SMs."""
    from fusedswiglu_b200 import _launch, _lib, parallel

    class Done:
        waited = 0

        def wait(self):
            Done.waited += 1

    T, dm, di = 2048, 512, 1536
    inp = orc.make_inputs(1, T, dm, di, "bf16", seed=6, dout_std=0.5)
    x = dev(inp["x"].reshape(T, dm), "bf16")
    dg = dev(inp["dout"].reshape(T, di), "bf16")
    du = dev((inp["dout"] * 0.5).reshape(T, di), "bf16")
    want_g, want_u = _launch.grad_weights(x, dg, du)
    monkeypatch.setattr(parallel, "plan_dw_split", lambda *a, **k: 512)
    got_g, got_u = parallel._CudaBackend.grad_weights_beside_collective(x, dg, du, world_size=4, work=Done())
    torch.cuda.synchronize()
    assert Done.waited == 1 and _lib.get_option("gemm_max_sms") == 0  # the cap was an argument, not an option
    assert torch.equal(got_g, want_g) and torch.equal(got_u, want_u)


# ------------------------------------- gate gradient inside the dX GEMM --
@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("T,dm,di", [(1000, 320, 1096), (2048, 512, 1536), (4224, 512, 2304), (130, 8, 8)])
def test_gate_gradient_inside_the_dx_gemm(T, dm, di, dtype):
    """The forward that saves s = silu(g) and t = u*silu'(g), and the dX GEMM whose warps
    produce dg = dout*t and du = dout*s on-chip: out is unchanged; s and t follow their
    formulas; the dg/du the kernel writes out are exactly dout*t and dout*s; dX is exactly
    the plain dX GEMM of those dg/du (same operand values, same accumulation order); and
    against the three-kernel path everything agrees to a rounding (the products are
    associated the other way round).  Ragged T, d_model and d_intermediate included."""
    from fusedswiglu_b200 import _launch, _lib

    inp = orc.make_inputs(1, T, dm, di, dtype, seed=T + di, dout_std=0.5)
    x, wg, wu = dev(inp["x"].reshape(T, dm), dtype), dev(inp["w_gate"], dtype), dev(inp["w_up"], dtype)
    dout = dev(inp["dout"].reshape(T, di), dtype)
    out0, g, u = _launch.forward(x, wg, wu, split_k=False)
    out1, s, t = _launch.forward(x, wg, wu, save_factors=True)
    assert torch.equal(out0, out1)
    gf = host(g).astype(np.float32)
    s_ref = orc.round16(orc.silu_f32(gf), dtype)
    t_ref = orc.round16(host(u) * orc.round16(orc.silu_grad_f32(gf), dtype), dtype)
    for name, got, want in (("s", s, s_ref), ("t", t, t_ref)):
        assert orc.rel_error(host(got), want) < 1e-3, name
        assert np.mean(orc.to_bits(host(got), dtype) != orc.to_bits(want, dtype)) < 0.02, name  # fast sigmoid
    dx, dg, du = _launch.grad_input_fused(dout, s, t, wg, wu)
    dg2, du2 = _launch.gate_grad_from_factors(dout, s, t)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.equal(dg, (dout.float() * t.float()).to(dout.dtype)) and torch.equal(dg, dg2)
    assert torch.equal(du, (dout.float() * s.float()).to(dout.dtype)) and torch.equal(du, du2)
    assert torch.equal(dx, _launch.grad_input(dg, du, wg, wu, split_k=False))
    # against the reference-order path
    dg0, du0 = _launch.gate_grad(dout, g, u)
    dx0 = _launch.grad_input(dg0, du0, wg, wu, split_k=False)
    assert torch.equal(du, du0)                      # du = dout * round(silu(g)) in both
    for name, a, b in (("dg", dg, dg0), ("dx", dx, dx0)):
        e = rel_error(a, b)
        print(f"fused gate gradient {dtype} T={T} {name}: rel_fro vs three-kernel path {e:.3e}")
        assert e < (4e-3 if dtype == "bf16" else 6e-4), (name, e)


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("T,dm,di", [(1000, 320, 1096), (4224, 512, 2304), (8200, 4096, 1536), (300, 64, 8)])
def test_gate_gradient_step_as_a_side_job_of_the_dx_kernel(T, dm, di, dtype):
    """fsw_backward_dx_gate: the elementwise step runs on the dX kernel's idle epilogue
    warps, in 2048-element quanta ahead of the tiles whose loads wait for their rows.  Same
    arithmetic, so dg, du and dX must be bit-identical to the two separate launches; six
    launches in a row go round the ring of control slots.  Ragged T (a partial last row
    tile), d_intermediate that is not a multiple of 64, several waves of tiles."""
    from fusedswiglu_b200 import _launch, _lib

    inp = orc.make_inputs(1, T, dm, di, dtype, seed=T + dm, dout_std=0.5)
    x, wg, wu = dev(inp["x"].reshape(T, dm), dtype), dev(inp["w_gate"], dtype), dev(inp["w_up"], dtype)
    dout = dev(inp["dout"].reshape(T, di), dtype)
    _, g, u = _launch.forward(x, wg, wu)
    dg0, du0 = _launch.gate_grad(dout, g, u)
    dx0 = _launch.grad_input(dg0, du0, wg, wu)
    for _ in range(6):
        dx, dg, du = _launch.gate_grad_and_input(dout, g, u, wg, wu)
        torch.cuda.synchronize()
        assert torch.equal(dg, dg0) and torch.equal(du, du0)
        assert torch.equal(dx, dx0)
    assert _lib.device_status() == 0


def test_fused_gate_gradient_mode_of_the_autograd_function():
    """FusedSwiGLU.fused_gate_grad = True on shapes of the reference's backward test,
    with its tolerance, against the PyTorch SwiGLU + autograd."""
    from fused_swiglu import FusedSwiGLU

    torch.manual_seed(0)
    worst = {}
    FusedSwiGLU.fused_gate_grad = True
    try:
        for bs, sq, dm, di in [(1, 64, 64, 64), (2, 128, 256, 512), (3, 192, 512, 1024), (4, 256, 1024, 2048),
                               (2, 512, 2048, 4096)]:
            x, wg, wu = make_input_weights(bs, sq, dm, di)
            dy = 0.1 * torch.randn(bs, sq, di, device="cuda", dtype=torch.bfloat16)
            x.requires_grad_(True), wg.requires_grad_(True), wu.requires_grad_(True)
            out = FusedSwiGLU.apply(x, wg, wu)
            out.backward(dy)
            got = {"out": out.detach(), "dx": x.grad, "dw_gate": wg.grad, "dw_up": wu.grad}
            xr, wgr, wur = (t.detach().clone().requires_grad_(True) for t in (x, wg, wu))
            ref = orc.swiglu_ref_torch(xr, wgr, wur)
            ref.backward(dy)
            want = {"out": ref.detach(), "dx": xr.grad, "dw_gate": wgr.grad, "dw_up": wur.grad}
            for k in got:
                e = rel_error(got[k], want[k])
                worst[k] = max(worst.get(k, 0.0), e)
                assert e < BFLOAT16_MAX_TOL, (bs, sq, dm, di, k, e)
    finally:
        FusedSwiGLU.fused_gate_grad = False
    print("fused gate gradient, worst rel error per tensor:", worst)


# ------------------------------------------------------------- fp16 paths --
@pytest.mark.parametrize("d_model", [1024, 2048])
def test_fp16_fast_accum_against_fp32_accum(d_model):
    """The fp16-accumulator variant is compared with the fp32-accumulate result,
    which the oracle pins; errors are reported per tensor."""
    bs, sq, di = 2, 512, 3 * d_model
    inp = orc.make_inputs(bs, sq, d_model, di, "fp16", seed=2, dout_std=0.1)
    slow = run_cuda(inp, "fp16", fast_accum=False)
    fast = run_cuda(inp, "fp16", fast_accum=True)
    for k in ("out", "dx", "dw_gate", "dw_up"):
        rep = orc.error_report(fast[k], slow[k])
        print(d_model, k, rep)
        assert np.all(np.isfinite(fast[k]))
        assert rep["rel_fro"] < BFLOAT16_MAX_TOL, (k, rep)


@pytest.mark.parametrize("d_model", [1024, 2048, 4096, 8192])
def test_fp16_fast_accum_sweep_at_full_size(d_model):
    """The fp16 sweep of the benchmark configurations: x (4, 2048, d_model),
    d_intermediate = 3*d_model, weights N(0, 1/d_model), dout = 0.1*randn; the
    fp16-accumulator run is compared with the fp32-accumulate run, per tensor."""
    from fusedswiglu_b200 import _launch

    T, di = 4 * 2048, 3 * d_model
    gen = torch.Generator(device="cuda").manual_seed(d_model)
    mk = lambda *s: torch.randn(*s, device="cuda", dtype=torch.float16, generator=gen)
    x, wg, wu = mk(T, d_model), mk(d_model, di) / math.sqrt(d_model), mk(d_model, di) / math.sqrt(d_model)
    dout = 0.1 * mk(T, di)
    res = {}
    for fast in (False, True):
        out, g, u = _launch.forward(x, wg, wu, fast_accum=fast)
        dg, du = _launch.gate_grad(dout, g, u)
        dx = _launch.grad_input(dg, du, wg, wu)
        dwg, dwu = _launch.grad_weights(x, dg, du, fast_accum=fast)
        res[fast] = {"out": out, "dx": dx, "dw_gate": dwg, "dw_up": dwu}
        del g, u, dg, du
    for k in ("out", "dx", "dw_gate", "dw_up"):
        a, b = res[True][k].float(), res[False][k].float()
        assert torch.all(torch.isfinite(a)), (d_model, k)
        e = (torch.linalg.norm(a - b) / torch.linalg.norm(b)).item()
        print(f"fp16 sweep d_model={d_model} {k}: rel_fro={e:.3e} max_abs={(a - b).abs().max().item():.3e}")
        assert e < BFLOAT16_MAX_TOL, (d_model, k, e)


def test_llama3_70b_shape_forward_only():
    """The largest configuration (16 x 4096 tokens, d_model 8192, d_intermediate
    28672) runs forward-only on one GPU: sampled rows against float64."""
    from fusedswiglu_b200 import _launch

    T, dm, di = 16 * 4096, 8192, 28672
    gen = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(T, dm, device="cuda", dtype=torch.bfloat16, generator=gen)
    wg = torch.randn(dm, di, device="cuda", dtype=torch.bfloat16, generator=gen) / math.sqrt(dm)
    wu = torch.randn(dm, di, device="cuda", dtype=torch.bfloat16, generator=gen) / math.sqrt(dm)
    out, _, _ = _launch.forward(x, wg, wu, save_activations=False)
    rows = torch.randint(0, T, (32,), device="cuda")
    g_ref = x[rows].double() @ wg.double()
    u_ref = x[rows].double() @ wu.double()
    assert rel_error(out[rows], torch.nn.functional.silu(g_ref) * u_ref) < EXPECTED_BF16
    # last tile rows and columns are written
    assert torch.all(torch.isfinite(out[-1].float())) and out[-1].abs().sum() > 0


def test_llama3_70b_column_shard_forward_and_backward():
    """One rank's share of the largest configuration when d_intermediate is split 8
    ways (16 x 4096 tokens, d_model 8192, 3584 local columns): forward + backward,
    per-tensor error against float64 on sampled rows and columns."""
    import bench
    from fusedswiglu_b200 import _launch

    T, dm, di_local = 16 * 4096, 8192, 28672 // 8
    x, wg, wu, dout = _full_size_inputs(T, dm, di_local, seed=11)
    out, g, u = _launch.forward(x, wg, wu)
    dg, du = _launch.gate_grad(dout, g, u)
    dx = _launch.grad_input(dg, du, wg, wu)
    dwg, dwu = _launch.grad_weights(x, dg, du)
    rep = bench.parity_report(x, wg, wu, dout, out, dx, dwg, dwu, world=1)
    for k in ("out", "dx", "dw_gate", "dw_up"):
        print(f"70B shard {k}: {rep[k]}")
        assert rep[k]["rel_fro"] < EXPECTED_BF16, (k, rep[k])


def test_fp16_accumulator_weight_gradient_over_32768_tokens():
    """The fp16 tensor-memory accumulator on the longest reduction of the benchmark
    configurations (32768 tokens): dW against the fp32-accumulate result and against
    float64, per tensor."""
    import bench
    from fusedswiglu_b200 import _launch

    T, dm, di = 32768, 2048, 2048
    gen = torch.Generator(device="cuda").manual_seed(12)
    mk = lambda *s: torch.randn(*s, device="cuda", dtype=torch.float16, generator=gen)
    x, wg, wu = mk(T, dm), mk(dm, di) / math.sqrt(dm), mk(dm, di) / math.sqrt(dm)
    dout = 0.1 * mk(T, di)
    out, g, u = _launch.forward(x, wg, wu)
    dg, du = _launch.gate_grad(dout, g, u)
    dx = _launch.grad_input(dg, du, wg, wu)
    slow = _launch.grad_weights(x, dg, du, fast_accum=False)
    fast = _launch.grad_weights(x, dg, du, fast_accum=True)
    for name, a, b in (("dw_gate", fast[0], slow[0]), ("dw_up", fast[1], slow[1])):
        assert torch.all(torch.isfinite(a.float())), name
        e = rel_error(a, b)
        print(f"fp16 accumulator over T={T}: {name} rel_fro vs fp32 accumulate = {e:.3e}")
        assert e < BFLOAT16_MAX_TOL, (name, e)
    rep = bench.parity_report(x, wg, wu, dout, out, dx, fast[0], fast[1], world=1)
    for k in ("out", "dx", "dw_gate", "dw_up"):
        print(f"fp16 accumulator over T={T}: {k} vs float64: {rep[k]}")
        assert rep[k]["rel_fro"] < BFLOAT16_MAX_TOL, (k, rep[k])


def test_fast_accum_function_matches_reference_semantics():
    from fused_swiglu import FastAccumFusedSwiGLU
    from fused_swiglu.kernels.kernels_fp16 import fused_swiglu_fwd

    torch.manual_seed(1)
    x, wg, wu = make_input_weights(2, 256, 512, 1024, dtype=torch.float16)
    ref = orc.swiglu_ref_torch(x, wg, wu)
    dy = 0.1 * torch.randn_like(ref)
    ref.backward(dy)
    want = [t.grad.clone() for t in (x, wg, wu)]
    x.grad, wg.grad, wu.grad = None, None, None
    out = FastAccumFusedSwiGLU.apply(x, wg, wu)
    out.backward(dy)
    assert rel_error(out, ref) < BFLOAT16_MAX_TOL
    for a, b in zip((x.grad, wg.grad, wu.grad), want):
        assert rel_error(a, b) < BFLOAT16_MAX_TOL
    o32, g32, u32 = fused_swiglu_fwd(x.detach(), wg.detach(), wu.detach(), fast_accum=False)
    assert rel_error(o32, ref) < EXPECTED_FP16
    assert rel_error(g32, x.detach() @ wg.detach()) < EXPECTED_FP16


# --------------------------------------------------- API surface behaviour --
def test_module_level_launchers_and_return_orders():
    from fused_swiglu.kernels.kernels_bf16 import elementwise_backward, fused_bmm, fused_swiglu_fwd

    torch.manual_seed(2)
    x, wg, wu = make_input_weights(3, 128, 192, 320)
    x, wg, wu = x.detach(), wg.detach(), wu.detach()
    out, g, u = fused_swiglu_fwd(x, wg, wu)
    assert out.shape == g.shape == u.shape == (3, 128, 320)
    assert rel_error(g, x @ wg) < EXPECTED_BF16 and rel_error(u, x @ wu) < EXPECTED_BF16
    dy = torch.randn_like(out)
    d_up, d_gate = elementwise_backward(dy, g, u)  # up first, like the reference
    gf = g.float()
    s = torch.sigmoid(gf)
    assert rel_error(d_up, dy.float() * gf * s) < 6e-3
    assert rel_error(d_gate, dy.float() * u.float() * (s + gf * s * (1 - s))) < 6e-3
    xT = x.transpose(1, 2)  # (bs, d_model, sq) strided view, as swiglu.py:51 passes
    gw_up, gw_gate = fused_bmm(xT, d_up, d_gate)
    assert gw_up.shape == (3, 192, 320)
    assert rel_error(gw_up, torch.bmm(xT.float(), d_up.float())) < EXPECTED_BF16
    assert rel_error(gw_gate, torch.bmm(xT.float(), d_gate.float())) < EXPECTED_BF16


def test_autocast_inputs_are_cast_like_custom_fwd():
    from fused_swiglu import FusedSwiGLU

    torch.manual_seed(3)
    x = torch.randn(1, 64, 128, device="cuda")
    wg = torch.randn(128, 256, device="cuda") / 11
    wu = torch.randn(128, 256, device="cuda") / 11
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = FusedSwiGLU.apply(x, wg, wu)
    assert out.dtype == torch.bfloat16
    ref = orc.swiglu_ref_torch(x.bfloat16(), wg.bfloat16(), wu.bfloat16())
    assert rel_error(out, ref) < EXPECTED_BF16


def test_non_contiguous_inputs_and_needs_input_grad():
    from fused_swiglu import FusedSwiGLU

    torch.manual_seed(4)
    xb = torch.randn(2, 64, 256, device="cuda", dtype=torch.bfloat16)
    x = xb[:, :, ::2].requires_grad_(False)  # strided, no grad
    wg = (torch.randn(128, 192, device="cuda", dtype=torch.bfloat16) / 11).requires_grad_(True)
    wu = (torch.randn(192, 128, device="cuda", dtype=torch.bfloat16) / 11).t().requires_grad_(True)  # strided
    out = FusedSwiGLU.apply(x, wg, wu)
    ref = orc.swiglu_ref_torch(x, wg.detach(), wu.detach())
    assert rel_error(out, ref) < EXPECTED_BF16
    out.sum().backward()
    assert wg.grad is not None and wg.grad.shape == wg.shape


# ------------------------------------------------------------- edge cases --
def _canary(shape, dtype, rows_pad=4):
    """Output buffer with guard rows before and after, filled with a sentinel."""
    full = torch.full((shape[0] + 2 * rows_pad, shape[1]), 777.0, device="cuda", dtype=dtype)
    return full, full[rows_pad:rows_pad + shape[0]]


@pytest.mark.parametrize("T,dm,di", [(1, 64, 64), (100, 72, 136), (257, 200, 520), (130, 8, 8), (64, 1032, 24)])
def test_edge_shapes_through_the_c_abi_with_guard_rows(T, dm, di):
    """Tokens not a multiple of any tile, feature sizes that are only multiples of
    8, and guard rows around every output to catch out-of-bounds stores."""
    from fusedswiglu_b200 import _lib

    lib = _lib.load()
    inp = orc.make_inputs(1, T, dm, di, "bf16", seed=T, dout_std=0.5)
    x, wg, wu = dev(inp["x"][0], "bf16"), dev(inp["w_gate"], "bf16"), dev(inp["w_up"], "bf16")
    dout = dev(inp["dout"][0], "bf16")
    bufs = {k: _canary(s, torch.bfloat16) for k, s in
            {"out": (T, di), "g": (T, di), "u": (T, di), "dg": (T, di), "du": (T, di), "dx": (T, dm),
             "dwg": (dm, di), "dwu": (dm, di)}.items()}
    v = {k: b[1] for k, b in bufs.items()}
    st = torch.cuda.current_stream().cuda_stream
    p = lambda t: t.data_ptr()
    _lib.check("fwd", lib.fsw_forward(p(x), p(wg), p(wu), p(v["out"]), p(v["g"]), p(v["u"]), T, dm, di, 0, 0, st))
    _lib.check("bwd", lib.fsw_backward(p(dout), p(x), p(wg), p(wu), p(v["g"]), p(v["u"]), p(v["dg"]), p(v["du"]),
                                       p(v["dx"]), p(v["dwg"]), p(v["dwu"]), T, dm, di, 0, 0, st))
    torch.cuda.synchronize()
    for k, (full, view) in bufs.items():
        assert torch.all(full[:4] == 777.0) and torch.all(full[-4:] == 777.0), f"{k}: guard rows overwritten"
        assert not torch.any(view == 777.0), f"{k}: elements left unwritten"
    out = orc.swiglu_ref(inp["x"], inp["w_gate"], inp["w_up"], "bf16")
    dxr, dwgr, dwur = orc.swiglu_ref_backward(inp["x"], inp["w_gate"], inp["w_up"], inp["dout"], "bf16")
    assert orc.rel_error(host(v["out"]), out[0]) < 1e-3
    assert orc.rel_error(host(v["dx"]), dxr[0]) < EXPECTED_BF16
    assert orc.rel_error(host(v["dwg"]), dwgr) < EXPECTED_BF16
    assert orc.rel_error(host(v["dwu"]), dwur) < EXPECTED_BF16


def test_empty_batch():
    from fused_swiglu import FusedSwiGLU

    x = torch.zeros(2, 0, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    wg = torch.ones(64, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    wu = torch.ones(64, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = FusedSwiGLU.apply(x, wg, wu)
    assert out.shape == (2, 0, 128)
    out.sum().backward()
    assert x.grad.shape == x.shape and torch.all(wg.grad == 0) and torch.all(wu.grad == 0)


def test_inference_mode_skips_saved_activations():
    from fusedswiglu_b200 import _launch

    inp = orc.make_inputs(1, 192, 128, 256, "bf16", seed=9)
    x, wg, wu = dev(inp["x"][0], "bf16"), dev(inp["w_gate"], "bf16"), dev(inp["w_up"], "bf16")
    out1, g, u = _launch.forward(x, wg, wu, save_activations=True)
    out2, g2, u2 = _launch.forward(x, wg, wu, save_activations=False)
    assert g2 is None and u2 is None and torch.equal(out1, out2)


def test_extreme_gate_values_stay_finite():
    from fusedswiglu_b200 import _launch

    x = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    x[:, 0] = torch.linspace(-300, 300, 64, device="cuda").bfloat16()
    wg = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    wg[0, :] = 1.0
    wu = wg.clone()
    out, g, u = _launch.forward(x, wg, wu)
    dg, du = _launch.gate_grad(torch.ones_like(out), g, u)
    for t in (out, dg, du):
        assert torch.all(torch.isfinite(t.float()))
    ref = torch.nn.functional.silu(g.float()) * u.float()
    assert rel_error(out, ref) < EXPECTED_BF16
    assert torch.all(out[0].float() == 0)  # silu(-300) * (-300) -> -0 * -300 = 0


# ------------------------------------- full-size, size-independent properties --
def _full_size_inputs(T, dm, di, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(T, dm, device="cuda", dtype=torch.bfloat16, generator=g)
    wg = torch.randn(dm, di, device="cuda", dtype=torch.bfloat16, generator=g) / math.sqrt(dm)
    wu = torch.randn(dm, di, device="cuda", dtype=torch.bfloat16, generator=g) / math.sqrt(dm)
    dout = torch.randn(T, di, device="cuda", dtype=torch.bfloat16, generator=g)
    return x, wg, wu, dout


@pytest.mark.parametrize("T,dm,di", [(8192, 4096, 12288), (32768, 4096, 14336)])
def test_full_size_properties(T, dm, di):
    """At the benchmark sizes: sampled rows/columns against fp64 dot products,
    exact linearity of the backward in dout (scaling by 2 is exact in floating
    point), and exact row-permutation equivariance of the forward."""
    from fusedswiglu_b200 import _launch

    x, wg, wu, dout = _full_size_inputs(T, dm, di)
    out, g, u = _launch.forward(x, wg, wu)
    rows = torch.randint(0, T, (64,), device="cuda")
    g_ref = x[rows].double() @ wg.double()
    u_ref = x[rows].double() @ wu.double()
    o_ref = torch.nn.functional.silu(g_ref) * u_ref
    assert rel_error(g[rows], g_ref) < EXPECTED_BF16
    assert rel_error(u[rows], u_ref) < EXPECTED_BF16
    assert rel_error(out[rows], o_ref) < EXPECTED_BF16

    dg, du = _launch.gate_grad(dout, g, u)
    dx = _launch.grad_input(dg, du, wg, wu)
    dwg, dwu = _launch.grad_weights(x, dg, du)
    dx_ref = dg[rows].double() @ wg.double().T + du[rows].double() @ wu.double().T
    assert rel_error(dx[rows], dx_ref) < EXPECTED_BF16
    cols = torch.randint(0, di, (32,), device="cuda")
    dwg_ref = x.double().T @ dg[:, cols].double()
    dwu_ref = x.double().T @ du[:, cols].double()
    assert rel_error(dwg[:, cols], dwg_ref) < EXPECTED_BF16
    assert rel_error(dwu[:, cols], dwu_ref) < EXPECTED_BF16

    # linearity: backward(2*dout) == 2*backward(dout), bit for bit
    dg2, du2 = _launch.gate_grad(dout * 2, g, u)
    assert torch.equal(dg2, dg * 2) and torch.equal(du2, du * 2)
    dx2 = _launch.grad_input(dg2, du2, wg, wu)
    assert torch.equal(dx2, dx * 2)
    dwg2, dwu2 = _launch.grad_weights(x, dg2, du2)
    assert torch.equal(dwg2, dwg * 2) and torch.equal(dwu2, dwu * 2)
    del dg2, du2, dx2, dwg2, dwu2

    # permutation equivariance: reversing the tokens reverses the output rows (without the
    # split of the last wave, which would add the K pieces of other tiles in another order)
    out1, _, _ = _launch.forward(x, wg, wu, save_activations=False, split_k=False)
    outp, _, _ = _launch.forward(x.flip(0).contiguous(), wg, wu, save_activations=False, split_k=False)
    assert torch.equal(outp.flip(0), out1)


# ------------------------------------------------- bounded waits, error path --
def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    """The TMA producer is told to issue nothing (a host-set test hook), so no
    barrier is ever signalled: the consumers' bounded waits run out after the
    (shortened) limit, the kernel records a status code, frees its tensor memory and
    returns.  Nothing faults or hangs; the next launch works normally."""
    from fusedswiglu_b200 import _launch, _lib

    inp = orc.make_inputs(1, 256, 128, 256, "bf16", seed=4)
    x, wg, wu = dev(inp["x"][0], "bf16"), dev(inp["w_gate"], "bf16"), dev(inp["w_up"], "bf16")
    assert _lib.device_status() == 0
    old_limit = _lib.get_option("wait_limit_ms")
    _lib.set_option("wait_limit_ms", 100)
    _lib.set_option("stall_producer", 1)
    try:
        _launch.forward(x, wg, wu)
        torch.cuda.synchronize()  # returns: the kernel gave up by itself
        with pytest.raises(_lib.FusedSwiGLUError) as err:
            _lib.check("fsw_status", -4 if _lib.load().fsw_status() != 0 else 0)
        assert "bounded wait" in str(err.value)
    finally:
        _lib.set_option("stall_producer", 0)
        _lib.set_option("wait_limit_ms", old_limit)
    assert _lib.device_status() == 0  # reading the status cleared it
    out, g, u = _launch.forward(x, wg, wu)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert orc.rel_error(host(out), orc.swiglu_ref(inp["x"], inp["w_gate"], inp["w_up"], "bf16")[0]) < 1e-3


# ------------------------------------------- memory mode, module, CUDA graphs --
def test_recompute_mode_gives_bit_identical_gradients():
    from fused_swiglu import FusedSwiGLU

    torch.manual_seed(7)
    x, wg, wu = make_input_weights(2, 320, 448, 832)
    dy = torch.randn(2, 320, 832, device="cuda", dtype=torch.bfloat16)
    grads = {}
    for mode in (False, True):
        FusedSwiGLU.recompute_activations = mode
        try:
            x.grad = wg.grad = wu.grad = None
            out = FusedSwiGLU.apply(x, wg, wu)
            saved = out.grad_fn.saved_tensors
            assert len(saved) == (3 if mode else 5)
            out.backward(dy)
            grads[mode] = (out.detach().clone(), x.grad.clone(), wg.grad.clone(), wu.grad.clone())
        finally:
            FusedSwiGLU.recompute_activations = False
    for a, b in zip(grads[False], grads[True]):
        assert torch.equal(a, b)


def test_nn_module_wrapper():
    from fusedswiglu_b200.nn import SwiGLU

    torch.manual_seed(8)
    m = SwiGLU(256, 512, device="cuda")
    x = torch.randn(2, 64, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = m(x)
    ref = orc.swiglu_ref_torch(x, m.w_gate, m.w_up)
    assert rel_error(out, ref) < EXPECTED_BF16
    out.float().pow(2).mean().backward()
    assert m.w_gate.grad.shape == (256, 512) and x.grad.shape == x.shape


def test_forward_backward_can_be_replayed_from_a_cuda_graph():
    """After one eager warm-up (which does the per-device set-up), a step can be
    captured in a CUDA graph and replayed on new inputs with identical results."""
    from fused_swiglu import FusedSwiGLU

    torch.manual_seed(9)
    bs, sq, dm, di = 1, 128, 512, 1536  # the launch-bound plumbing shape
    wg = (torch.randn(dm, di, device="cuda", dtype=torch.bfloat16) / math.sqrt(dm)).requires_grad_(True)
    wu = (torch.randn(dm, di, device="cuda", dtype=torch.bfloat16) / math.sqrt(dm)).requires_grad_(True)
    static_x = torch.randn(bs, sq, dm, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    static_dy = torch.randn(bs, sq, di, device="cuda", dtype=torch.bfloat16)

    def step():
        out = FusedSwiGLU.apply(static_x, wg, wu)
        gx, gg, gu = torch.autograd.grad(out, (static_x, wg, wu), static_dy)
        return out, gx, gg, gu

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_out = step()
    for seed in (1, 2):
        gen = torch.Generator(device="cuda").manual_seed(seed)
        with torch.no_grad():
            static_x.copy_(torch.randn(bs, sq, dm, device="cuda", dtype=torch.bfloat16, generator=gen))
            static_dy.copy_(torch.randn(bs, sq, di, device="cuda", dtype=torch.bfloat16, generator=gen))
        graph.replay()
        torch.cuda.synchronize()
        replayed = [t.clone() for t in static_out]
        eager = step()
        for a, b in zip(replayed, eager):
            assert torch.equal(a, b)

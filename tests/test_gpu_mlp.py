"""The plain tcgen05 GEMM entry point (fsw_gemm) and the SwiGLU MLP block built
on it, against PyTorch on the same GPU."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-2          # the reference's bound on the relative Frobenius error
EXPECTED = 6e-3


def rel(a, b):
    return (torch.linalg.norm(a.float() - b.float()) / torch.linalg.norm(b.float())).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(64, 64, 64), (100, 72, 136), (257, 520, 200), (1024, 1536, 1024),
                                   (3000, 4096, 1800), (8, 8, 8)])
def test_gemm_three_layouts_match_a_float64_product(M, N, K, dtype):
    from fusedswiglu_b200 import _launch, _lib

    gen = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", dtype=dtype, generator=gen)
    b = torch.randn(K, N, device="cuda", dtype=dtype, generator=gen) / math.sqrt(K)
    want = (a.double() @ b.double())
    c_nn = _launch.gemm(a, b)
    c_nt = _launch.gemm(a, b.t().contiguous(), trans_b=True) if K % 8 == 0 else None
    c_tn = _launch.gemm(a.t().contiguous(), b, trans_a=True) if M % 8 == 0 else None
    torch.cuda.synchronize()
    bound = 2.5e-3 if dtype == torch.bfloat16 else 4e-4   # one rounding of an exact-ish sum
    for name, c in (("nn", c_nn), ("nt", c_nt), ("tn", c_tn)):
        if c is None:
            continue
        assert c.shape == (M, N)
        assert rel(c, want) < bound, (name, rel(c, want))
    # the three layouts accumulate K in the same order: identical bits
    if c_nt is not None:
        assert torch.equal(c_nn, c_nt)
    if c_tn is not None:
        assert torch.equal(c_nn, c_tn)
    assert _lib.device_status() == 0


def test_gemm_argument_errors():
    from fusedswiglu_b200 import _launch, _lib

    a = torch.zeros(16, 12, device="cuda", dtype=torch.bfloat16)   # K = 12 is not a multiple of 8
    b = torch.zeros(12, 16, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(_lib.FusedSwiGLUError, match="multiples of 8"):
        _launch.gemm(a, b)
    with pytest.raises(AssertionError, match="Dimension mismatch"):
        _launch.gemm(torch.zeros(16, 16, device="cuda", dtype=torch.bfloat16), b)


@pytest.mark.parametrize("shape", [(2, 192, 256, 704, 256), (1, 1000, 512, 1536, 384)])
def test_mlp_block_forward_backward(shape):
    from fusedswiglu_b200.mlp import FusedSwiGLUMLP, SwiGLUMLP

    bs, sq, dm, di, do = shape
    torch.manual_seed(sum(shape))
    m = SwiGLUMLP(dm, di, do, device="cuda")
    x = torch.randn(bs, sq, dm, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(bs, sq, do, device="cuda", dtype=torch.bfloat16)

    ref = (torch.nn.functional.silu(x @ m.w_gate) * (x @ m.w_up)) @ m.w_down
    ref.backward(dy)
    want = [ref.detach()] + [t.grad.clone() for t in (x, m.w_gate, m.w_up, m.w_down)]
    x.grad = None
    m.zero_grad(set_to_none=True)

    y = m(x)
    y.backward(dy)
    got = [y.detach(), x.grad, m.w_gate.grad, m.w_up.grad, m.w_down.grad]
    for name, a, b in zip(("y", "dx", "dw_gate", "dw_up", "dw_down"), got, want):
        assert a.shape == b.shape
        e = rel(a, b)
        print(shape, name, e)
        assert e < TOL and e < EXPECTED, (name, e)


@pytest.mark.parametrize("layout", ["nn", "nt", "tn"])
def test_plain_gemm_with_a_split_last_wave(layout):
    """fsw_gemm_ws: 9 x 10 = 90 tiles are one wave of 74 plus 16 tiles whose K loops
    (128 blocks) are divided over all SM pairs.  Deterministic, and within a rounding of
    both the unsplit launch and a float64 product."""
    from fusedswiglu_b200 import _launch, _lib

    M, N, K = 2300, 5000, 8192
    gen = torch.Generator(device="cuda").manual_seed(7)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, generator=gen)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16, generator=gen) / math.sqrt(K)
    if layout == "nn":
        run = lambda **kw: _launch.gemm(a, b, **kw)
    elif layout == "nt":
        bt = b.t().contiguous()
        run = lambda **kw: _launch.gemm(a, bt, trans_b=True, **kw)
    else:
        at = a[:2296].t().contiguous()  # a row length must be a multiple of 8
        run = lambda **kw: _launch.gemm(at, b, trans_a=True, **kw)
    plain, s1, s2 = run(split_k=False), run(), run()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    want = (a[:plain.shape[0]].double() @ b.double())
    assert torch.equal(s1, s2)
    assert int((s1 != plain).sum()) > 0          # the split did run
    assert rel(s1, plain) < 1e-3
    assert rel(s1, want) < 1.05 * rel(plain, want) + 1e-5

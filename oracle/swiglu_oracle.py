"""CPU restatement of the reference's SwiGLU algorithm.  TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA path: only tests/, the smoke check and
the bench's CPU-baseline leg may import it.  Nothing in the product package
imports it, and the product has no CPU path.

Two restatements, both in numpy with explicit 16-bit rounding points:

  * ``swiglu_ref`` / ``swiglu_ref_backward`` follow the reference's own oracle,
    ``swiglu_ref_torch`` + autograd (fused_swiglu/test_swiglu.py:47-55, 96-103):
    every PyTorch op rounds its result to the tensor dtype.
  * ``kernel_forward`` / ``kernel_elementwise_backward`` / ``kernel_backward``
    follow the rounding order of the reference's Triton kernels and autograd
    Function (fused_swiglu/kernels/kernels_bf16.py:102-160, 210-234, 343-382;
    fused_swiglu/swiglu.py:34-58).

``swiglu_ref_torch`` is the same three-line formula on torch tensors; it is what
the bench times on the host cores.

Pinning: tests/golden/*.npz were produced by running the reference's own
``swiglu_ref_torch`` (imported from the reference checkout) on CPU, see
tests/golden/make_golden.py; tests/test_oracle.py checks this module against them.
GEMMs accumulate in float64 here, so results equal an fp32-accumulate GEMM up to
the last bit of the 16-bit rounding.  The fp16-ACCUMULATE variant of the
reference (kernels_fp16.py:69-75, 318-319) depends on tensor-core internals and
has no reference test: for it parity is unpinned, and the tests compare against
the fp32-accumulate result instead.
"""
from __future__ import annotations

from typing import Dict, Tuple

import numpy as np

DTYPES = ("bf16", "fp16")


# ----------------------------------------------------------------- rounding --
def round_bf16(a: np.ndarray) -> np.ndarray:
    """float32 -> nearest bfloat16 (ties to even), returned as float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    lsb = (bits >> 16) & 1
    rounded = ((bits + 0x7FFF + lsb) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    nan = np.isnan(a)
    if nan.any():
        out = np.where(nan, np.float32(np.nan), out)
    return out.reshape(a.shape)


def round_fp16(a: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        return np.asarray(a, dtype=np.float32).astype(np.float16).astype(np.float32)


def round16(a: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "bf16":
        return round_bf16(a)
    if dtype == "fp16":
        return round_fp16(a)
    raise ValueError(f"unknown dtype {dtype!r}")


def to_bits(a: np.ndarray, dtype: str) -> np.ndarray:
    """16-bit storage pattern (uint16) of values already rounded to `dtype`."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    if dtype == "bf16":
        return (a.view(np.uint32) >> 16).astype(np.uint16)
    return a.astype(np.float16).view(np.uint16)


def from_bits(b: np.ndarray, dtype: str) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    if dtype == "bf16":
        return (b.astype(np.uint32) << 16).view(np.float32)
    return b.view(np.float16).astype(np.float32)


# -------------------------------------------------------------- elementwise --
def sigmoid_f32(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    with np.errstate(over="ignore"):
        return (np.float32(1) / (np.float32(1) + np.exp(-x, dtype=np.float32))).astype(np.float32)


def silu_f32(x: np.ndarray) -> np.ndarray:
    """x * sigmoid(x) in fp32 (kernels_bf16.py:9-11 before its cast)."""
    return (np.asarray(x, np.float32) * sigmoid_f32(x)).astype(np.float32)


def silu_grad_f32(x: np.ndarray) -> np.ndarray:
    """sigmoid(x) + x*sigmoid(x)*(1-sigmoid(x)) in fp32 (kernels_bf16.py:14-16)."""
    x = np.asarray(x, np.float32)
    s = sigmoid_f32(x)
    return (s + x * s * (np.float32(1) - s)).astype(np.float32)


def _mm(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """GEMM of 16-bit-valued operands with a wide accumulator, result in fp32."""
    return (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)


def rel_error(x: np.ndarray, y: np.ndarray) -> float:
    """||x - y||_F / ||y||_F (test_swiglu.py:43-44)."""
    x = np.asarray(x, np.float64)
    y = np.asarray(y, np.float64)
    return float(np.linalg.norm(x - y) / np.linalg.norm(y))


def error_report(x: np.ndarray, y: np.ndarray) -> Dict[str, float]:
    """rel-Frobenius, max-abs and max-rel error of x against y."""
    x = np.asarray(x, np.float64)
    y = np.asarray(y, np.float64)
    d = np.abs(x - y)
    denom = np.maximum(np.abs(y), 1e-6 * max(float(np.abs(y).max(initial=0.0)), 1e-30))
    return {
        "rel_fro": float(np.linalg.norm(x - y) / max(np.linalg.norm(y), 1e-30)),
        "max_abs": float(d.max(initial=0.0)),
        "max_rel": float((d / denom).max(initial=0.0)),
    }


# ------------------------------------------- the reference's PyTorch oracle --
def swiglu_ref(x: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray, dtype: str = "bf16") -> np.ndarray:
    """silu(x @ w_gate) * (x @ w_up) with one rounding per op (test_swiglu.py:47-55).

    x is (..., d_model); weights are (d_model, d_intermediate)."""
    g = round16(_mm(x.reshape(-1, x.shape[-1]), w_gate), dtype)
    u = round16(_mm(x.reshape(-1, x.shape[-1]), w_up), dtype)
    s = round16(silu_f32(g), dtype)
    out = round16(s * u, dtype)
    return out.reshape(*x.shape[:-1], w_gate.shape[1])


def swiglu_from_saved(g: np.ndarray, u: np.ndarray, dtype: str = "bf16") -> np.ndarray:
    """out from the 16-bit g = x@w_gate and u = x@w_up, with the rounding points of
    ``silu(x_gate) * x_up`` on 16-bit tensors (test_swiglu.py:52-55): silu evaluated
    in fp32 and rounded, then the product rounded."""
    return round16(round16(silu_f32(g), dtype) * u, dtype)


def swiglu_ref_backward(
    x: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray, dy: np.ndarray, dtype: str = "bf16"
) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(dX, dW_gate, dW_up) as autograd computes them for ``swiglu_ref`` with
    16-bit leaf tensors (test_swiglu.py:96-103): mul backward, silu backward
    evaluated in fp32 from the 16-bit g, two matmul backwards each rounded, and
    the two contributions to dX added in 16 bits."""
    x2 = x.reshape(-1, x.shape[-1])
    dy2 = dy.reshape(-1, dy.shape[-1])
    g = round16(_mm(x2, w_gate), dtype)
    u = round16(_mm(x2, w_up), dtype)
    s = round16(silu_f32(g), dtype)
    d_s = round16(dy2 * u, dtype)
    d_u = round16(dy2 * s, dtype)
    sg = sigmoid_f32(g)
    d_g = round16(d_s * (sg * (np.float32(1) + g * (np.float32(1) - sg))), dtype)
    dx = round16(round16(_mm(d_g, w_gate.T), dtype) + round16(_mm(d_u, w_up.T), dtype), dtype)
    dwg = round16(_mm(x2.T, d_g), dtype)
    dwu = round16(_mm(x2.T, d_u), dtype)
    return dx.reshape(x.shape), dwg, dwu


# ---------------------------------------------- the reference's kernel order --
def kernel_forward(
    x: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray, dtype: str = "bf16"
) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(out, g, u) with the rounding order of swiglu_kernel with fp32 accumulators
    (kernels_bf16.py:143-160; kernels_fp16.py:152-169 with fast_accum=False):
    g and u are the rounded accumulators; out = round(u_acc * round(silu(g_acc)))."""
    x2 = x.reshape(-1, x.shape[-1])
    g_acc = _mm(x2, w_gate)
    u_acc = _mm(x2, w_up)
    out = round16(u_acc * round16(silu_f32(g_acc), dtype), dtype)
    shape = (*x.shape[:-1], w_gate.shape[1])
    return out.reshape(shape), round16(g_acc, dtype).reshape(shape), round16(u_acc, dtype).reshape(shape)


def kernel_elementwise_backward(
    dout: np.ndarray, g: np.ndarray, u: np.ndarray, dtype: str = "bf16"
) -> Tuple[np.ndarray, np.ndarray]:
    """(grad_xw_up, grad_xw_gate) - up first - as elementwise_backward_kernel
    computes them (kernels_bf16.py:228-234): du = dout * round(silu(g)),
    dg = round(dout * u) * round(silu'(g)), each product rounded."""
    du = round16(dout * round16(silu_f32(g), dtype), dtype)
    dg = round16(round16(dout * u, dtype) * round16(silu_grad_f32(g), dtype), dtype)
    return du, dg


def kernel_backward(
    x: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray, g: np.ndarray, u: np.ndarray, dout: np.ndarray,
    dtype: str = "bf16",
) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(dX, dW_gate, dW_up) following FusedSwiGLU.backward (swiglu.py:34-58) for
    x (bs, sq, d_model): two rounded GEMMs and a 16-bit add for dX (:45), per-batch
    rounded weight gradients (kernels_bf16.py:366,381) summed in 16 bits (:11-13)."""
    bs = x.shape[0]
    du, dg = kernel_elementwise_backward(dout, g, u, dtype)
    dg2 = dg.reshape(-1, dg.shape[-1])
    du2 = du.reshape(-1, du.shape[-1])
    dx = round16(round16(_mm(dg2, w_gate.T), dtype) + round16(_mm(du2, w_up.T), dtype), dtype)
    dwg = np.zeros(w_gate.shape, np.float32)
    dwu = np.zeros(w_up.shape, np.float32)
    for b in range(bs):
        dwg = round16(dwg + round16(_mm(x[b].T, dg[b]), dtype), dtype)
        dwu = round16(dwu + round16(_mm(x[b].T, du[b]), dtype), dtype)
    return dx.reshape(x.shape), dwg, dwu


# -------------------------------------------------------------------- inputs --
def make_inputs(
    bs: int, sq: int, d_model: int, d_intermediate: int, dtype: str = "bf16", seed: int = 0,
    dout_std: float = 1.0,
) -> Dict[str, np.ndarray]:
    """Seeded synthetic tensors with the reference's distributions
    (test_swiglu.py:23-40, 98): x ~ N(0,1), W ~ N(0,1)/sqrt(d_model), dout ~
    N(0, dout_std^2), each rounded to `dtype` and returned as float32.  One
    generator draws x, w_gate, w_up, dout in that order."""
    rng = np.random.default_rng(seed)
    x = round16(rng.standard_normal((bs, sq, d_model), dtype=np.float32), dtype)
    scale = np.float32(1.0 / np.sqrt(d_model))
    w_gate = round16(round16(rng.standard_normal((d_model, d_intermediate), dtype=np.float32), dtype) * scale, dtype)
    w_up = round16(round16(rng.standard_normal((d_model, d_intermediate), dtype=np.float32), dtype) * scale, dtype)
    dout = round16(np.float32(dout_std) * rng.standard_normal((bs, sq, d_intermediate), dtype=np.float32), dtype)
    return {"x": x, "w_gate": w_gate, "w_up": w_up, "dout": dout}


def reference_test_shapes(num_test: int = 3, seed: int = 0):
    """The (bs, sq, d_model, d_intermediate) lists the reference's two
    parametrised tests draw at import (test_swiglu.py:10-11, 58-67, 81-90):
    legacy numpy seed, nested comprehensions whose inner draws are repeated for
    every outer value, forward list first, then the backward list."""
    rs = np.random.RandomState(seed)

    def draw():
        return [
            (int(b), int(sq), int(dm), int(di))
            for b in rs.randint(1, 4, size=num_test)
            for sq in 64 * rs.randint(1, 32, size=num_test)
            for dm in 64 * rs.randint(1, 128, size=num_test)
            for di in 64 * rs.randint(1, 128, size=num_test)
        ]

    fwd = draw()
    bwd = draw()
    return fwd, bwd


# ------------------------------------------------- torch form (timed on CPU) --
def swiglu_ref_torch(x, w_gate, w_up):
    """The reference's PyTorch SwiGLU (test_swiglu.py:47-55) on torch tensors of
    any device/dtype; autograd gives its backward."""
    import torch

    return torch.nn.functional.silu(torch.matmul(x, w_gate)) * torch.matmul(x, w_up)

"""Generates tests/golden/*.npz by running the REFERENCE's own PyTorch oracle,
``swiglu_ref_torch`` (fused_swiglu/test_swiglu.py:47-55 of fattorib/fusedswiglu),
on CPU with autograd, exactly as its backward test does (test_swiglu.py:96-103).

Usage (needs the reference checkout; run from the repository root):

    python tests/golden/make_golden.py /path/to/fusedswiglu

Inputs come from oracle.swiglu_oracle.make_inputs (seeded numpy), so the fixtures
can be re-derived; tensors are stored as uint16 bit patterns.  For the larger
case only a hash of the seeded weights and every 16th row of the weight
gradients are stored, to keep the files small.
"""
from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent

# (name, bs, sq, d_model, d_intermediate, dtype, dout_std, compact)
CASES = [
    ("tiny_bf16", 1, 64, 64, 64, "bf16", 1.0, False),
    ("ragged_bf16", 2, 96, 192, 320, "bf16", 0.1, False),
    ("tiny_fp16", 2, 64, 128, 192, "fp16", 0.1, False),
    ("plumbing_bf16", 1, 128, 512, 1536, "bf16", 1.0, True),  # the CPU-runnable config
    ("plumbing_fp16", 1, 128, 512, 1536, "fp16", 0.1, True),
]
ROW_STEP = 16


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/fusedswiglu")
    ref_root = sys.argv[1]
    sys.path.insert(0, str(REPO))
    from oracle import swiglu_oracle as orc

    # The reference package must win the name `fused_swiglu` in this process.
    sys.path.insert(0, ref_root)
    import torch
    from fused_swiglu.test_swiglu import swiglu_ref_torch  # the reference's function

    assert str(Path(sys.modules["fused_swiglu"].__file__).resolve()).startswith(str(Path(ref_root).resolve()))
    tdt = {"bf16": torch.bfloat16, "fp16": torch.float16}

    for name, bs, sq, dm, di, dtype, dstd, compact in CASES:
        inp = orc.make_inputs(bs, sq, dm, di, dtype=dtype, seed=0, dout_std=dstd)
        t = {k: torch.from_numpy(v).to(tdt[dtype]) for k, v in inp.items()}
        x = t["x"].clone().requires_grad_(True)
        wg = t["w_gate"].clone().requires_grad_(True)
        wu = t["w_up"].clone().requires_grad_(True)
        out = swiglu_ref_torch(x, wg, wu)
        out.backward(t["dout"])
        res = {"out": out.detach(), "dx": x.grad, "dw_gate": wg.grad, "dw_up": wu.grad}
        res = {k: v.float().numpy() for k, v in res.items()}
        blob = {
            "meta": np.array([bs, sq, dm, di], dtype=np.int64),
            "dtype": np.array(dtype),
            "dout_std": np.array(dstd, dtype=np.float64),
            "seed": np.array(0, dtype=np.int64),
            "row_step": np.array(ROW_STEP if compact else 1, dtype=np.int64),
            "x": orc.to_bits(inp["x"], dtype),
            "dout": orc.to_bits(inp["dout"], dtype),
            "out": orc.to_bits(res["out"], dtype),
            "dx": orc.to_bits(res["dx"], dtype),
        }
        if compact:
            blob["w_gate_sha256"] = np.array(sha(orc.to_bits(inp["w_gate"], dtype)))
            blob["w_up_sha256"] = np.array(sha(orc.to_bits(inp["w_up"], dtype)))
            blob["dw_gate"] = orc.to_bits(res["dw_gate"][::ROW_STEP], dtype)
            blob["dw_up"] = orc.to_bits(res["dw_up"][::ROW_STEP], dtype)
        else:
            blob["w_gate"] = orc.to_bits(inp["w_gate"], dtype)
            blob["w_up"] = orc.to_bits(inp["w_up"], dtype)
            blob["dw_gate"] = orc.to_bits(res["dw_gate"], dtype)
            blob["dw_up"] = orc.to_bits(res["dw_up"], dtype)
        path = HERE / f"{name}.npz"
        np.savez_compressed(path, **blob)
        print(f"{path.name}: {path.stat().st_size / 1024:.0f} KiB, torch {torch.__version__}")


if __name__ == "__main__":
    main()

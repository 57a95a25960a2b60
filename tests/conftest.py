import os
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device of compute capability 10.x (B200)")


@pytest.fixture(scope="session", autouse=True)
def built_library():
    """The shared library is built once per session if it is missing or stale
    (nvcc cross-compiles without a GPU)."""
    from fusedswiglu_b200 import build

    if build.is_stale():
        build.build()
    return build.LIB_PATH


def load_golden(name):
    import numpy as np

    from oracle import swiglu_oracle as orc

    z = np.load(GOLDEN_DIR / f"{name}.npz")
    dtype = str(z["dtype"])
    bs, sq, dm, di = (int(v) for v in z["meta"])
    case = {"name": name, "dtype": dtype, "shape": (bs, sq, dm, di), "row_step": int(z["row_step"]),
            "dout_std": float(z["dout_std"]), "seed": int(z["seed"])}
    for k in ("x", "dout", "out", "dx", "dw_gate", "dw_up"):
        case[k] = orc.from_bits(z[k], dtype)
    if "w_gate" in z.files:
        case["w_gate"] = orc.from_bits(z["w_gate"], dtype)
        case["w_up"] = orc.from_bits(z["w_up"], dtype)
    else:
        import hashlib

        inp = orc.make_inputs(bs, sq, dm, di, dtype=dtype, seed=case["seed"], dout_std=case["dout_std"])
        for k in ("w_gate", "w_up"):
            digest = hashlib.sha256(orc.to_bits(inp[k], dtype).tobytes()).hexdigest()
            if digest != str(z[f"{k}_sha256"]):
                raise RuntimeError(
                    f"seeded {k} for golden case {name} does not reproduce on this numpy; "
                    "regenerate with tests/golden/make_golden.py"
                )
            case[k] = inp[k]
    return case


GOLDEN_CASES = ["tiny_bf16", "ragged_bf16", "tiny_fp16", "plumbing_bf16", "plumbing_fp16"]

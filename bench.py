#!/usr/bin/env python
"""Benchmark of the fused SwiGLU hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one forward + backward pass of the SwiGLU MLP block over one batch
of seeded synthetic tensors: the forward dual GEMM, the gate-gradient elementwise
kernel, the dX GEMM and the dW dual GEMM.  FLOPs are counted as 2*M*N*K per GEMM,
six GEMMs: 12*T*d_model*d_intermediate per step; elementwise work is not counted.

With N > 1 (launched by torch.distributed.run, one rank per GPU) d_intermediate is
sharded column-parallel and the timed loop IS the package's multi-GPU API
(ColumnParallelSwiGLU forward + backward): forward and dW are local, the partial
dX is all-reduced with NCCL while the dW GEMM runs.  The total problem is fixed,
so scaling is "strong".

After the timed region (outside it) every run checks its own results, per tensor,
against float64 on sampled rows and columns and puts the figures into the JSON line
(`parity`); a relative error above 1e-2 fails the run.

`--impl reference` times the reference path's PyTorch SwiGLU (forward + autograd
backward) on the host CPU cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

# name -> (bs, sq, d_model, d_intermediate, dtype)
WORKLOADS = {
    "llama3_8b_mlp": (8, 4096, 4096, 14336, "bf16"),
    "readme": (4, 2048, 4096, 12288, "bf16"),
    "llama3_70b_mlp": (16, 4096, 8192, 28672, "bf16"),
    "plumbing": (1, 128, 512, 1536, "bf16"),
    # fp16 sweep with the fp16 tensor-memory accumulator (FastAccumFusedSwiGLU): d_intermediate = 3*d_model
    "fp16_d1024": (4, 2048, 1024, 3072, "fp16"),
    "fp16_d2048": (4, 2048, 2048, 6144, "fp16"),
    "fp16_d4096": (4, 2048, 4096, 12288, "fp16"),
    "fp16_d8192": (4, 2048, 8192, 24576, "fp16"),
}
DEFAULT_WORKLOAD = "llama3_8b_mlp"
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}
PARITY_BOUND = 1e-2  # the reference's bound on ||a-b||_F/||b||_F (fused_swiglu/test_swiglu.py:20)
# DRAM bytes per launch from ncu captures (dram__bytes_read.sum + dram__bytes_write.sum),
# keyed "kernel/workload/n_gpus"; absent = not captured for that case.
DRAM_TRAFFIC_FILE = REPO / "profiles" / "dram_traffic_per_launch.json"

CLOCK_QUERY = (
    "timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
    "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
    "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preheat", type=float, default=3.0, metavar="SECONDS",
                    help="run the same step loop for this long before the warm-up steps, so that short timed "
                         "regions (many GPUs) are measured at the power-capped clock like long ones")
    ap.add_argument("--comm-ctas", type=int, default=16, metavar="N",
                    help="N>1: CTAs NCCL may use for the dX collective (= SMs the dW GEMM leaves free beside it); "
                         "0 = NCCL's own choice on the default group with the default reservation")
    ap.add_argument("--dx-collective", default="peer", choices=["peer", "peer-copy", "nccl"],
                    help="N>1: reduce dX with this library's kernels over NVLink peer memory (PeerDxReducer; "
                         "peer = partial sums stored to their owners from the GEMM epilogue, peer-copy = by copy "
                         "engines) or with NCCL beside the dW GEMM")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-gpu-bar", action="store_true",
                    help="skip timing torch's own CUDA SwiGLU (cuBLAS + eager kernels) on the same GPU")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--fp32-accum", action="store_true",
                    help="fp16 workloads: accumulate in fp32 instead of the fp16 accumulator")
    ap.add_argument("--opt", action="append", default=[], metavar="NAME=VALUE",
                    help="library tuning knob passed to fsw_set_option, e.g. --opt group_m=16 (repeatable)")
    ap.add_argument("--only", default=None, choices=["fwd", "ew", "dx", "dw", "fwdst", "dxf", "mlp"],
                    help="launch only this kernel in each step (for profiling one kernel); prints no bench line")
    ap.add_argument("--shard-of", type=int, default=1, metavar="N",
                    help="with --only on one GPU: time rank 0's 1/N column shard of the workload")
    return ap.parse_args()


def load_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def load_dram_traffic(kernel, workload, world):
    try:
        return json.loads(DRAM_TRAFFIC_FILE.read_text()).get(f"{kernel}/{workload}/{world}")
    except Exception:
        return None


def host_threads():
    """Host threads this process may use (torch.distributed.run exports
    OMP_NUM_THREADS=1, which must not decide the CPU baseline's thread count)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


# ------------------------------------------------------------ clock sampling --
REASON_BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))


# Runs in a child process (its own interpreter: polling must not compete with the
# bench's launch loop for the GIL): NVML queries every 4 ms, one CSV line per sample.
NVML_POLLER = r"""
import sys, time
import pynvml
uuid, index, path = sys.argv[1], int(sys.argv[2]), sys.argv[3]
pynvml.nvmlInit()
try:
    h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
except Exception:
    h = pynvml.nvmlDeviceGetHandleByIndex(index)
with open(path, "w", buffering=1) as f:
    f.write("max,%d\n" % pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
    while True:
        try:
            f.write("%.6f,%d,%.3f,%d\n" % (time.time(), pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM),
                                          pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0,
                                          pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)))
        except Exception:
            pass
        time.sleep(0.004)
"""


class ClockSampler:
    """Samples SM clock, power and clock-event reasons while a region runs: NVML
    polled every few milliseconds by a child process (read-only queries, the ones
    nvidia-smi makes), or, if NVML cannot be loaded, an nvidia-smi loop."""

    def __init__(self, gpu_uuid: str, index: int):
        self.uuid, self.index = gpu_uuid, index
        self.rows = []  # (host time, sm MHz, power W, reasons bitmask)
        self.max_mhz = None
        self._nvml = None
        self._nvml_path = None
        self._smi = None
        self._smi_path = None
        self.source = None

    def start(self):
        import tempfile

        try:
            import pynvml  # noqa: F401  (only to know that the child can import it)

            fd, self._nvml_path = tempfile.mkstemp(prefix="fsw_clocks_", suffix=".csv")
            os.close(fd)
            self._nvml = subprocess.Popen([sys.executable, "-c", NVML_POLLER, self.uuid or "", str(self.index),
                                           self._nvml_path], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
            time.sleep(0.5)
            if self._nvml.poll() is None and os.path.getsize(self._nvml_path) > 0:
                self.source = "nvml from a child process, 4 ms period"
                return
            self._nvml.kill()
        except Exception:
            pass
        self._nvml = None
        fd, self._smi_path = tempfile.mkstemp(prefix="fsw_clocks_", suffix=".csv")
        os.close(fd)
        try:
            self._smi = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", self.uuid or str(self.index)],
                stdout=open(self._smi_path, "w"), stderr=subprocess.DEVNULL)
            self.source = "nvidia-smi -lms 20"
        except OSError:
            self._smi = None

    def _finish(self):
        if self._nvml is not None:
            self._nvml.terminate()
            try:
                self._nvml.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._nvml.kill()
            self._nvml = None
            for line in Path(self._nvml_path).read_text().splitlines():
                f = line.split(",")
                try:
                    if f[0] == "max":
                        self.max_mhz = float(f[1])
                    elif len(f) == 4:
                        self.rows.append((float(f[0]), float(f[1]), float(f[2]), int(f[3])))
                except ValueError:
                    continue
            os.unlink(self._nvml_path)
        if self._smi is not None:
            import datetime

            self._smi.terminate()
            try:
                self._smi.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._smi.kill()
            self._smi = None
            for line in Path(self._smi_path).read_text().splitlines():
                f = [s.strip() for s in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    mask = sum(bit for i, (_, bit) in enumerate(REASON_BITS) if f[5 + i].lower().startswith("active"))
                    self.rows.append((ts, float(f[1]), float(f[3]), mask))
                    self.max_mhz = float(f[2])
                except ValueError:
                    continue
            os.unlink(self._smi_path)

    def summary(self, t_begin, t_end, label):
        """Median SM clock and the reasons seen among the samples taken in [t_begin, t_end]."""
        self._finish()
        rows = [r for r in self.rows if t_begin <= r[0] <= t_end]
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": len(rows), "window": label,
               "source": self.source}
        if rows:
            sm = sorted(r[1] for r in rows)
            out.update(sm_mhz=sm[len(sm) // 2], sm_mhz_min=sm[0], sm_mhz_max=sm[-1],
                       reasons=[n for n, bit in REASON_BITS if any(r[3] & bit for r in rows)],
                       power_w_max=max(r[2] for r in rows))
        return out


def flops_per_step(T, dm, di):
    return 12.0 * T * dm * di


# ------------------------------------------------------------ reference arm --
def cpu_sample_tokens(T, dm, di):
    """Tokens per CPU step: the whole workload when that is at most ~25 TFLOP of
    work (a few seconds on a host of this class), else the largest T/2^k that is."""
    t = T
    while flops_per_step(t, dm, di) > 25e12 and t % 2 == 0 and t > 1024:
        t //= 2
    return t


def cpu_reference_run(bs, sq, dm, di, dtype, steps, warmup, sample_tokens, seed=0):
    """The reference path's PyTorch SwiGLU + autograd (fused_swiglu/test_swiglu.py:47-55,
    96-103) on the host cores, over `sample_tokens` tokens of the workload per step."""
    import torch

    from oracle import swiglu_oracle as orc

    threads = host_threads()
    torch.set_num_threads(threads)
    tdt = {"bf16": torch.bfloat16, "fp16": torch.float16}[dtype]
    T = min(sample_tokens, bs * sq)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(1, T, dm, generator=g).to(tdt).requires_grad_(True)
    wg = (torch.randn(dm, di, generator=g) / dm ** 0.5).to(tdt).requires_grad_(True)
    wu = (torch.randn(dm, di, generator=g) / dm ** 0.5).to(tdt).requires_grad_(True)
    dout = torch.randn(1, T, di, generator=g).to(tdt)

    def step():
        x.grad = wg.grad = wu.grad = None
        out = orc.swiglu_ref_torch(x, wg, wu)
        out.backward(dout)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return {"tokens": T, "sec_per_step": dt, "tflops": flops_per_step(T, dm, di) / dt / 1e12,
            "threads": torch.get_num_threads()}


def cpu_baseline_object(r, T, steps, warmup):
    import torch

    whole = r["tokens"] == T
    return {"value": r["tflops"], "unit": "TFLOP/s", "cores": r["threads"], "kind": "port",
            "sample": (f"the whole workload ({T} tokens) per step" if whole else
                       f"{r['tokens']} of {T} tokens per step") +
                      f", {steps} step(s) after {warmup} warm-up, {r['sec_per_step']:.2f} s per step; the reference's "
                      f"PyTorch SwiGLU + autograd restated in oracle/ (the reference's own module needs its Triton "
                      f"import chain and is not on this machine), torch {torch.__version__} CPU, "
                      f"{r['threads']} threads of os.cpu_count()={os.cpu_count()}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return

    bs, sq, dm, di, dtype = WORKLOADS[args.workload]
    T = bs * sq
    sample = cpu_sample_tokens(T, dm, di)
    steps = max(1, min(args.steps, 3))
    warmup = 1
    r = cpu_reference_run(bs, sq, dm, di, dtype, steps, warmup, sample, args.seed)
    line = {
        "impl": "reference",
        "metric": "swiglu_fwd_bwd_tflops", "value": r["tflops"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": r["sec_per_step"] * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": args.workload, "bs": bs, "sq": sq, "d_model": dm, "d_intermediate": di,
                   "sample_tokens_per_step": r["tokens"], "device": "host CPU"},
        "cpu_baseline": cpu_baseline_object(r, T, steps, warmup),
        "e2e": {"value": r["tflops"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "fwd_tokens_per_s": None,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------- parity --
class _Err:
    """Running error figures of one tensor over several sampled blocks."""

    def __init__(self):
        self.num = self.den = 0.0
        self.max_abs = self.max_rel = self.ref_max = 0.0
        self.pending = []

    def add(self, got, ref):
        d = (got.double() - ref).abs()
        self.num += float((d * d).sum())
        self.den += float((ref * ref).sum())
        self.max_abs = max(self.max_abs, float(d.max()))
        self.ref_max = max(self.ref_max, float(ref.abs().max()))
        self.pending.append((d, ref.abs()))

    def reduce(self, dist, world, dev):
        import torch

        if world > 1:
            t = torch.tensor([self.num, self.den], device=dev, dtype=torch.float64)
            dist.all_reduce(t)
            self.num, self.den = float(t[0]), float(t[1])
            m = torch.tensor([self.max_abs, self.ref_max], device=dev, dtype=torch.float64)
            dist.all_reduce(m, op=dist.ReduceOp.MAX)
            self.max_abs, self.ref_max = float(m[0]), float(m[1])
        # max-rel with max(|ref|, 1e-6 * max|ref|) as denominator (near-zero entries dominate it)
        floor = 1e-6 * self.ref_max
        for d, r in self.pending:
            self.max_rel = max(self.max_rel, float((d / r.clamp_min(floor)).max())) if floor > 0 else self.max_rel
        if world > 1:
            m = torch.tensor([self.max_rel], device=dev, dtype=torch.float64)
            dist.all_reduce(m, op=dist.ReduceOp.MAX)
            self.max_rel = float(m[0])
        self.pending = []
        return {"rel_fro": (self.num / self.den) ** 0.5 if self.den > 0 else 0.0, "max_abs": self.max_abs,
                "max_rel": self.max_rel}


def parity_report(x2d, wg, wu, dout2d, out, dx, dwg, dwu, world, seed=1234, n_rows=64, n_cols=32):
    """Per-tensor error of this run's results against float64 on sampled rows (out,
    dX) and sampled columns (dW_gate, dW_up).  Collective: with world > 1 every rank
    calls it; out and dW are checked on each rank's own columns, dX (all-reduced, the
    same on every rank) against the float64 sum of the ranks' partial products."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    dev = x2d.device
    T, dm = x2d.shape
    di_local = wg.shape[1]
    gen = torch.Generator().manual_seed(seed)  # CPU generator: the same rows on every rank
    rows = torch.randperm(T, generator=gen)[:min(n_rows, T)].to(dev)
    cols = torch.randperm(di_local, generator=gen)[:min(n_cols, di_local)].to(dev)
    wg64, wu64 = wg.double(), wu.double()
    errs = {k: _Err() for k in ("out", "dx", "dw_gate", "dw_up")}

    xr = x2d[rows].double()
    g, u = xr @ wg64, xr @ wu64
    errs["out"].add(out[rows], F.silu(g) * u)
    s = torch.sigmoid(g)
    d = dout2d[rows].double()
    dg, du = d * u * (s + g * s * (1 - s)), d * g * s
    dx_ref = dg @ wg64.T + du @ wu64.T
    if world > 1:
        dist.all_reduce(dx_ref)
    errs["dx"].add(dx[rows], dx_ref)
    del wg64, wu64, g, u, s, d, dg, du

    wgc, wuc = wg[:, cols].double(), wu[:, cols].double()
    acc_g = torch.zeros(dm, cols.numel(), device=dev, dtype=torch.float64)
    acc_u = torch.zeros_like(acc_g)
    for r0 in range(0, T, 4096):
        xc = x2d[r0:r0 + 4096].double()
        g, u = xc @ wgc, xc @ wuc
        s = torch.sigmoid(g)
        d = dout2d[r0:r0 + 4096][:, cols].double()
        acc_g += xc.T @ (d * u * (s + g * s * (1 - s)))
        acc_u += xc.T @ (d * g * s)
    errs["dw_gate"].add(dwg[:, cols], acc_g)
    errs["dw_up"].add(dwu[:, cols], acc_u)
    rep = {k: e.reduce(dist, world, dev) for k, e in errs.items()}
    rep["reference"] = (f"float64 SwiGLU + gradient formulas on {rows.numel()} sampled rows (out, dX) and "
                        f"{cols.numel()} sampled columns per rank (dW_gate, dW_up)")
    rep["bound"] = PARITY_BOUND
    rep["ok"] = all(rep[k]["rel_fro"] < PARITY_BOUND for k in errs)
    return rep


# ------------------------------------------------------------------ our arm --
def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N>1 must be launched with torch.distributed.run (one rank per GPU)")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from fusedswiglu_b200 import FastAccumFusedSwiGLU, FusedSwiGLU, _launch, _lib, parallel

    # The dX collective runs on a group whose NCCL kernels are capped to as many CTAs
    # as the dW GEMM leaves SMs free for them.
    use_peer = world > 1 and args.dx_collective in ("peer", "peer-copy")
    group = (parallel.new_collective_group(max_ctas=args.comm_ctas)
             if world > 1 and args.comm_ctas > 0 and not use_peer else None)

    _lib.load()
    for item in args.opt:
        name, _, value = item.partition("=")
        _lib.set_option(name, int(value))
    bs, sq, dm, di, dtype = WORKLOADS[args.workload]
    tdt = {"bf16": torch.bfloat16, "fp16": torch.float16}[dtype]
    fast = dtype == "fp16" and not args.fp32_accum  # fp16 accumulator in forward and dW
    FastAccumFusedSwiGLU.fast_accum = fast
    T = bs * sq
    if args.shard_of > 1:
        if not args.only or world != 1:
            raise SystemExit("--shard-of needs --only and a single GPU")
        lo, hi = parallel.shard_bounds(di, 0, args.shard_of)
    else:
        lo, hi = parallel.shard_bounds(di, rank, world)
    di_local = hi - lo
    K, W = args.steps, max(args.warmup, 3)

    # Seeded synthetic tensors; every rank draws the full tensors from one seed and
    # keeps its column slice, so the sharded run computes the same problem.
    g = torch.Generator(device=dev).manual_seed(args.seed)
    x = torch.randn(bs, sq, dm, device=dev, dtype=tdt, generator=g)
    wg_full = torch.randn(dm, di, device=dev, dtype=tdt, generator=g) / dm ** 0.5
    wu_full = torch.randn(dm, di, device=dev, dtype=tdt, generator=g) / dm ** 0.5
    wg = wg_full[:, lo:hi].contiguous()
    wu = wu_full[:, lo:hi].contiguous()
    del wg_full, wu_full
    dout_full = torch.randn(bs, sq, di, device=dev, dtype=tdt, generator=g)
    dout = dout_full[..., lo:hi].contiguous() if world > 1 or args.shard_of > 1 else dout_full
    del dout_full
    if dtype == "fp16":
        dout *= 0.1  # the reference's dy = 0.1 * randn (test_swiglu.py:98)
    x2d = x.view(T, dm)
    dout2d = dout.view(T, di_local)

    names = ["fwd_dual_gemm", "gate_grad_elementwise", "dx_gemm", "dw_dual_gemm"]
    launches = {"n": 0}
    dw_split = {"first": None, "collective_ms": None}

    def counted(fn):
        def wrapper(*a, **kw):
            launches["n"] += 1
            return fn(*a, **kw)
        return wrapper

    # Every C-ABI kernel launch goes through these functions; count them.
    for _name in ("forward", "gate_grad", "grad_input", "grad_weights", "grad_input_scatter", "reduce_dx_slices",
                  "wait_flags"):
        setattr(_launch, _name, counted(getattr(_launch, _name)))

    class Marked:
        """The product backend with a labelled CUDA event recorded before each launch;
        the time from one event to the next is charged to the first one's label."""
        marks = None  # list of (label, event) of the step being timed, or None
        pool = []     # events created before the timed region

        @staticmethod
        def mark(label):
            if Marked.marks is not None:
                e = Marked.pool.pop() if Marked.pool else torch.cuda.Event(enable_timing=True)
                e.record()
                Marked.marks.append((label, e))

        @staticmethod
        def forward(*a, **kw):
            Marked.mark("fwd_dual_gemm")
            return _launch.forward(*a, **kw)

        @staticmethod
        def gate_grad(*a, **kw):
            Marked.mark("gate_grad_elementwise")
            return _launch.gate_grad(*a, **kw)

        @staticmethod
        def grad_input(*a, **kw):
            Marked.mark("dx_gemm")
            return _launch.grad_input(*a, **kw)

        @staticmethod
        def grad_weights(*a, **kw):
            Marked.mark("dw_dual_gemm")
            r = _launch.grad_weights(*a, **kw)
            Marked.mark("after_dw")
            return r

        @staticmethod
        def grad_weights_beside_collective(x2d_, dg, du, **kw):
            Marked.mark("dw_dual_gemm")
            if dw_split["first"] is None and kw.get("work") is not None:
                dw_split["collective_ms"] = (kw.get("collective_s") or 0.0) * 1e3
                dw_split["first"] = parallel.plan_dw_split(
                    x2d_.shape[0], x2d_.shape[1], dg.shape[1], kw.get("world_size", world),
                    _lib.get_option("sm_count"), parallel.comm_sms(world, kw.get("group")), x2d_.element_size(),
                    kw.get("collective", "all_reduce"), kw.get("collective_s"))
            r = parallel._CudaBackend.grad_weights_beside_collective(x2d_, dg, du, **kw)
            Marked.mark("after_dw")
            return r

    wgp = wg.clone().requires_grad_(True)
    wup = wu.clone().requires_grad_(True)

    reducer = None
    if use_peer:
        # Symmetric memory needs peer access between all GPUs of the job; if it cannot be set
        # up on every rank, all ranks fall back to NCCL together.
        try:
            real_reducer = parallel.PeerDxReducer(T, dm, tdt, dev, group,
                                                  scatter="copy" if args.dx_collective == "peer-copy" else "epilogue")
            ok = torch.ones(1, device=dev)
        except Exception as exc:  # noqa: BLE001
            real_reducer, ok = None, torch.zeros(1, device=dev)
            print(f"rank {rank}: peer-memory reduction unavailable ({type(exc).__name__}: {exc}); using NCCL",
                  file=sys.stderr, flush=True)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) == 0.0:
            real_reducer, use_peer = None, False
            group = parallel.new_collective_group(max_ctas=args.comm_ctas) if args.comm_ctas > 0 else None
    if use_peer:

        class MarkedReducer:
            """The product's reducer with the same labelled events."""
            columns_before_reduction = staticmethod(real_reducer.columns_before_reduction)

            @staticmethod
            def scatter(*a, **kw):
                Marked.mark("dx_gemm")
                return real_reducer.scatter(*a, **kw)

            @staticmethod
            def reduce(*a, **kw):
                Marked.mark("dx_reduction")
                r = real_reducer.reduce(*a, **kw)
                Marked.mark("after_dw")
                return r

        reducer = MarkedReducer
        dw_split["first"] = real_reducer.columns_before_reduction(di_local, False)

    def step(marks=None):
        """One forward + backward.  world == 1: the launch sequence of FusedSwiGLU
        (the autograd Function adds nothing on the device).  world > 1: the package's
        ColumnParallelSwiGLU forward and backward themselves."""
        Marked.marks = marks
        if world == 1:
            out, gg, uu = Marked.forward(x2d, wg, wu, fast_accum=fast)
            dg, du = Marked.gate_grad(dout2d, gg, uu)
            dx = Marked.grad_input(dg, du, wg, wu)
            dwg, dwu = Marked.grad_weights(x2d, dg, du, fast_accum=fast)
            Marked.mark("end")
            Marked.marks = None
            return out, dx, dwg, dwu
        xin = x.detach().requires_grad_(True)
        wgp.grad = wup.grad = None
        out = parallel.column_parallel_swiglu(xin, wgp, wup, group=group, fast_accum=fast, backend=Marked,
                                              reducer=reducer)
        out.backward(dout)
        Marked.mark("end")
        Marked.marks = None
        return out.detach().view(T, di_local), xin.grad.view(T, dm), wgp.grad, wup.grad

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.only == "mlp":
        # The whole MLP block (SwiGLU + down projection, forward + backward) on this
        # library against torch's (cuBLAS + eager elementwise) on the same GPU, alternating.
        from fusedswiglu_b200.mlp import FusedSwiGLUMLP

        xm = x.detach().clone().requires_grad_(True)
        wgm, wum = (w_.detach().clone().requires_grad_(True) for w_ in (wg, wu))
        wdm = (torch.randn(di_local, dm, device=dev, dtype=tdt, generator=g) / di_local ** 0.5).requires_grad_(True)
        dy = torch.randn(bs, sq, dm, device=dev, dtype=tdt, generator=g)

        def ours():
            xm.grad = wgm.grad = wum.grad = wdm.grad = None
            FusedSwiGLUMLP.apply(xm, wgm, wum, wdm).backward(dy)

        def lib():
            xm.grad = wgm.grad = wum.grad = wdm.grad = None
            ((torch.nn.functional.silu(xm @ wgm) * (xm @ wum)) @ wdm).backward(dy)

        t0 = time.time()
        while time.time() - t0 < args.preheat:
            ours()
            torch.cuda.synchronize()
        res = {"this_library": [], "torch": []}
        for _ in range(4):
            for name, fn in (("this_library", ours), ("torch", lib)):
                for _ in range(3):
                    fn()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(K):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                res[name].append(e0.elapsed_time(e1) / K)
        flops = 18.0 * T * dm * di_local
        med = {k: sorted(v)[len(v) // 2] for k, v in res.items()}
        print(json.dumps({"only": "mlp", "workload": args.workload, "flops_per_step": flops,
                          "ms": med, "tflops": {k: flops / v / 1e9 for k, v in med.items()},
                          "status": _lib.device_status()}), flush=True)
        return

    if args.only:
        # Profiling aid: the other kernels run once to produce this kernel's inputs.
        out, gg, uu = _launch.forward(x2d, wg, wu, fast_accum=fast)
        dg, du = _launch.gate_grad(dout2d, gg, uu)
        one = {
            "fwd": lambda: _launch.forward(x2d, wg, wu, fast_accum=fast),
            "ew": lambda: _launch.gate_grad(dout2d, gg, uu),
            "dx": lambda: _launch.grad_input(dg, du, wg, wu),
            "dw": lambda: _launch.grad_weights(x2d, dg, du, fast_accum=fast),
            # the gate gradient inside the dX GEMM: forward that saves silu(g) and u*silu'(g), fused dX
            "fwdst": lambda: _launch.forward(x2d, wg, wu, fast_accum=fast, save_factors=True),
            "dxf": None,
        }[args.only]
        if args.only == "dxf":
            _, sf, tf = _launch.forward(x2d, wg, wu, fast_accum=fast, save_factors=True)
            one = lambda: _launch.grad_input_fused(dout2d, sf, tf, wg, wu)
        for _ in range(W):
            one()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(K):
            one()
        t1.record()
        barrier()
        ms = t0.elapsed_time(t1) / K
        print(json.dumps({"only": args.only, "workload": args.workload, "ms": ms, "steps": K,
                          "tflops": (4.0 * T * dm * di_local / ms / 1e9) if args.only != "ew" else None,
                          "sm_khz": _lib.get_option("last_sm_khz"),
                          "status": _lib.device_status()}), flush=True)
        return

    props = torch.cuda.get_device_properties(dev)
    gpu_id = str(getattr(props, "uuid", ""))
    if gpu_id and not gpu_id.startswith("GPU-"):
        gpu_id = "GPU-" + gpu_id
    sampler = ClockSampler(gpu_id, local_rank)
    if rank == 0:
        sampler.start()
    # Pre-heat: the same step loop for a fixed wall time, so that the timed region of
    # every GPU count starts at the clock the power cap settles at.
    barrier()
    pre0 = time.time()
    pre_steps = 0
    while True:
        for _ in range(4):
            step()
            pre_steps += 1
        torch.cuda.synchronize()
        flag = torch.tensor([1.0 if time.time() - pre0 < args.preheat else 0.0], device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)  # all ranks leave together
        if float(flag.item()) == 0.0:
            break
    for _ in range(W):
        step()
    barrier()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches["n"] = 0
    step_marks = [[] for _ in range(K)]
    Marked.pool = [torch.cuda.Event(enable_timing=True) for _ in range(12 * K)]
    kernels0 = _lib.get_option("kernel_launches")
    wall0 = time.time()
    t_start.record()
    for i in range(K):
        step(step_marks[i])
    t_end.record()
    barrier()
    wall1 = time.time()
    n_launches = _lib.get_option("kernel_launches") - kernels0  # counted inside the library, second passes included
    clocks = None
    if rank == 0:
        clocks = sampler.summary(wall0, wall1, "timed region")
        pre = ClockSampler.summary(sampler, pre0, wall0, "pre-heat and warm-up (same step loop)")
        clocks["before_timed_region"] = {k: pre[k] for k in ("sm_mhz", "reasons", "samples", "window")}
    total_ms = t_start.elapsed_time(t_end)
    by_label = {}
    for marks in step_marks:
        for (label, e0), (_, e1) in zip(marks, marks[1:]):
            by_label[label] = by_label.get(label, 0.0) + e0.elapsed_time(e1) / K
    per_kernel_ms = [by_label.get(n, 0.0) for n in names]
    # "after_dw": between the end of a dW launch and whatever follows it - at the end of
    # the step that is the part of the collective left exposed
    tail_ms = by_label.get("after_dw", 0.0)
    reduction_ms = by_label.get("dx_reduction")
    # per-rank view: GPUs of one box differ by several percent under the power cap, and the
    # one collective of the step makes every rank wait for the slowest
    per_rank = None
    if world > 1:
        labels = names + ["dx_reduction", "after_dw"]
        mine = torch.tensor([by_label.get(n, 0.0) for n in labels], device=dev, dtype=torch.float64)
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        per_rank = {n: [round(float(t[i]), 4) for t in allr] for i, n in enumerate(labels)}
    if world > 1:
        tt = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        total_ms = float(tt.item())
    status = _lib.device_status()
    if status != 0:
        raise SystemExit(f"a kernel gave up on a bounded wait (status {status}); no number reported")
    pacing = {"pace_kb": _lib.get_option("pace_kb"), "switched_off_in_last_launch": _lib.get_option("pace_off")}
    ms_per_step = total_ms / K
    total_flops = flops_per_step(T, dm, di)  # whole job, all ranks
    value = total_flops / ms_per_step / 1e9

    # ---- parity of what the timed loop computed (outside the timed region)
    parity = None
    if not args.no_parity:
        out_c, dx_c, dwg_c, dwu_c = step()
        torch.cuda.synchronize()
        parity = parity_report(x2d, wg, wu, dout2d, out_c, dx_c, dwg_c, dwu_c, world)
        dx_keep_for_e2e = dx_c
        del out_c, dwg_c, dwu_c
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps({"error": "parity check failed", "parity": parity}), flush=True)
            raise SystemExit(f"results differ from float64 by more than {PARITY_BOUND}: {parity}")
    else:
        dx_keep_for_e2e = None

    # ---- end to end through the public autograd API with host buffers
    e2e = None
    if not args.no_e2e:
        # world > 1: the tokens are sharded at the boundary as well (row_sharded mode):
        # a rank uploads its T/world rows of x and its column shard of dout, and
        # downloads the reduce-scattered dX of its own rows.
        rs = world > 1 and bs % world == 0
        b_mine = bs // world if rs else bs
        x_src = x[rank * b_mine:(rank + 1) * b_mine] if rs else x
        hx = torch.empty_like(x_src, device="cpu").pin_memory()
        hdout = torch.empty_like(dout, device="cpu").pin_memory()
        hx.copy_(x_src)
        hdout.copy_(dout)
        hdx = torch.empty_like(x_src, device="cpu").pin_memory()
        wgp.grad = wup.grad = None
        # Double-buffered input pipeline, as a training loop's loader would run it:
        # while step i computes, the copy stream uploads step i+1's x and dout into
        # the other buffer set and a third stream downloads step i-1's dX.  Every
        # step still moves all of its inputs from the host and its result back.
        h2d_stream = torch.cuda.Stream(device=dev)
        d2h_stream = torch.cuda.Stream(device=dev)
        x_dev = [torch.empty_like(x_src) for _ in range(2)]
        dout_dev = [torch.empty_like(dout) for _ in range(2)]
        dx_keep = [None, None]
        ready = [None, None]       # inputs of buffer b are on the device
        consumed = [None, None]    # the step that used buffer b has finished
        downloaded = [None, None]  # dX of buffer b has been copied out
        state = {"i": 0}

        def upload(b):
            with torch.cuda.stream(h2d_stream):
                if consumed[b] is not None:
                    h2d_stream.wait_event(consumed[b])
                x_dev[b].copy_(hx, non_blocking=True)
                dout_dev[b].copy_(hdout, non_blocking=True)
                ready[b] = torch.cuda.Event()
                ready[b].record()

        def e2e_step():
            main = torch.cuda.current_stream(dev)
            b = state["i"] & 1
            if ready[b] is None:
                upload(b)
            main.wait_event(ready[b])
            upload(b ^ 1)  # next step's inputs, overlapped with this step's compute
            xin = x_dev[b].detach().requires_grad_(True)
            wgp.grad = wup.grad = None
            if world > 1:
                out = parallel.column_parallel_swiglu(xin, wgp, wup, group=group, fast_accum=fast, row_sharded=rs,
                                                      reducer=real_reducer if use_peer else None)
            elif dtype == "fp16":
                out = FastAccumFusedSwiGLU.apply(xin, wgp, wup)
            else:
                out = FusedSwiGLU.apply(xin, wgp, wup)
            out.backward(dout_dev[b])
            done = torch.cuda.Event()
            done.record()
            consumed[b] = done
            ready[b] = None
            dx_keep[b] = xin.grad
            with torch.cuda.stream(d2h_stream):
                d2h_stream.wait_event(done)
                hdx.copy_(dx_keep[b], non_blocking=True)
                downloaded[b] = torch.cuda.Event()
                downloaded[b].record()
            main.wait_event(downloaded[b ^ 1]) if downloaded[b ^ 1] is not None else None
            state["i"] += 1

        def e2e_drain():
            for evt in downloaded:
                if evt is not None:
                    torch.cuda.current_stream(dev).wait_event(evt)

        for _ in range(3):
            e2e_step()
        barrier()
        n_e2e = max(3, min(K, 10))
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(n_e2e):
            e2e_step()
        e2e_drain()
        s1.record()
        barrier()
        e2e_ms = s0.elapsed_time(s1) / n_e2e
        if world > 1:
            tt = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e2e_ms = float(tt.item())
        # the dX that came back to the host against the device-resident run's
        dx_host_rel = None
        if dx_keep_for_e2e is not None:
            want = dx_keep_for_e2e.view(bs, sq, dm)[rank * b_mine:(rank + 1) * b_mine] if rs else dx_keep_for_e2e.view(bs, sq, dm)
            got = hdx.to(dev)
            dx_host_rel = float(torch.linalg.norm(got.float() - want.float()) / torch.linalg.norm(want.float()))
            if world > 1:
                tt = torch.tensor([dx_host_rel], device=dev, dtype=torch.float64)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                dx_host_rel = float(tt.item())
            if not dx_host_rel < PARITY_BOUND:
                raise SystemExit(f"end-to-end dX differs from the device-resident run's by {dx_host_rel}")
        if world == 1:
            api = ("FastAccumFusedSwiGLU" if dtype == "fp16" else "FusedSwiGLU") + ".apply + backward"
            note = ("every step uploads its x and dout from pinned host memory and downloads its dX; uploads for "
                    "step i+1 and the download of step i overlap step i's kernels (double-buffered); weights "
                    "stay resident")
        else:
            api = f"column_parallel_swiglu(row_sharded={rs}) + backward"
            note = (("tokens sharded at the boundary: every step each rank uploads its T/N rows of x and its column "
                     "shard of dout from pinned host memory, all-gathers x over NVLink, and downloads its T/N rows "
                     "of the reduce-scattered dX; ") if rs else
                    "every step each rank uploads the whole x and its column shard of dout and downloads the whole "
                    "all-reduced dX; ") + \
                "uploads for step i+1 and the download of step i overlap step i's kernels (double-buffered); " \
                "weights stay resident; bytes are per rank"
        e2e = {"value": total_flops / e2e_ms / 1e9, "unit": "TFLOP/s",
               "h2d_bytes_per_step": hx.numel() * 2 + hdout.numel() * 2, "d2h_bytes_per_step": hdx.numel() * 2,
               "ms_per_step": e2e_ms, "steps": n_e2e, "api": api, "note": note,
               "dx_rel_to_device_resident_run": dx_host_rel}
        status = _lib.device_status()
        if status != 0:
            raise SystemExit(f"a kernel gave up on a bounded wait (status {status}) in the end-to-end loop")
        del x_dev, dout_dev, dx_keep
    del dx_keep_for_e2e

    # ---- same-box bar: the reference test's oracle expression on this GPU through
    # torch (two cuBLAS GEMMs + eager silu/mul, autograd backward).  Library code, timed
    # after everything above so that it cannot disturb the numbers reported as ours.
    gpu_bar = None
    if world == 1 and not args.no_gpu_bar:
        xr = x.detach().clone().requires_grad_(True)
        wgr = wg.detach().clone().requires_grad_(True)
        wur = wu.detach().clone().requires_grad_(True)

        def bar_step():
            xr.grad = wgr.grad = wur.grad = None
            o = torch.nn.functional.silu(xr @ wgr) * (xr @ wur)
            o.backward(dout)

        for _ in range(3):
            bar_step()
        n_bar = max(3, min(K, 10))
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        b0.record()
        for _ in range(n_bar):
            bar_step()
        b1.record()
        torch.cuda.synchronize()
        bar_ms = b0.elapsed_time(b1) / n_bar
        gpu_bar = {"value": total_flops / bar_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": bar_ms, "steps": n_bar,
                   "what": "torch CUDA silu(x@W_gate)*(x@W_up) + autograd backward on the same GPU "
                           "(cuBLAS GEMMs + eager elementwise kernels); a library bar, not this repo's code"}
        del xr, wgr, wur

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_src = load_peaks()
    gemm_flops_local = 4.0 * T * dm * di_local
    kern = {}
    for j, n in enumerate(names):
        ms = per_kernel_ms[j]
        if n == "gate_grad_elementwise":
            gbs = 5.0 * T * di_local * 2 / ms / 1e6
            kern[n] = {"ms": ms, "achieved": gbs, "unit": "GB/s", "bound": "hbm", "frac": gbs / peaks["hbm_gbs"]}
        else:
            tf = gemm_flops_local / ms / 1e9
            kern[n] = {"ms": ms, "achieved": tf, "unit": "TFLOP/s", "bound": "tensor",
                       "frac": tf / peaks["bf16_tflops_sustained"]}
    if world > 1 and use_peer:
        kern["dx_gemm"]["note"] = ("the GEMM's epilogue stores the partial sums into the owning ranks' buffers "
                                   "over NVLink")
        kern["dx_reduction"] = {"ms": reduction_ms, "note": "waits (time-limited) for the peers' partials, adds the "
                                                            "slices in fp32; queued between two column ranges of dW"}
        kern["dw_dual_gemm"]["note"] = ("all SMs, in two column ranges around the reduction; copy engines gather "
                                        "the reduced row blocks beside the second")
        kern["collective_exposed_after_dw"] = {"ms": tail_ms}
    elif world > 1:
        kern["dw_dual_gemm"]["note"] = ("runs beside the NCCL all-reduce of dX; first column range on "
                                        f"{_lib.get_option('sm_count') - parallel.comm_sms(world, group)} SMs")
        kern["collective_exposed_after_dw"] = {"ms": tail_ms}
    dom = max((n for n in names if n != "gate_grad_elementwise"), key=lambda n: kern[n]["ms"])
    roofline = {
        "kernel": dom, "bound": "tensor", "achieved": kern[dom]["achieved"], "peak": peaks["bf16_tflops_sustained"],
        "unit": "TFLOP/s", "frac": kern[dom]["achieved"] / peaks["bf16_tflops_sustained"],
        "peak_source": f"{peak_src} bf16_tflops_sustained (kernel timed inside a long step)",
        "frac_of_burst": kern[dom]["achieved"] / peaks["bf16_tflops"],
        "frac_of_nominal": kern[dom]["achieved"] / NOMINAL_BF16_TFLOPS,
        "algorithmic_flops_per_launch": gemm_flops_local,
        "traffic": load_dram_traffic(dom, args.workload, world),
        "algorithmic_hbm_bytes_per_launch": {
            "fwd_dual_gemm": 2.0 * (T * dm + 2 * dm * di_local + 3 * T * di_local),
            "dx_gemm": 2.0 * (2 * T * di_local + 2 * dm * di_local + T * dm),
            "dw_dual_gemm": 2.0 * (T * dm + 2 * T * di_local + 2 * dm * di_local),
        }[dom],
        "kernels": kern,
    }
    fwd_tokens_per_s = T / (per_kernel_ms[0] / 1e3)

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        tokens = cpu_sample_tokens(T, dm, di)
        r = cpu_reference_run(bs, sq, dm, di, dtype, steps=2, warmup=1, sample_tokens=tokens, seed=args.seed)
        cpu_baseline = cpu_baseline_object(r, T, 2, 1)

    sm_mhz = clocks.get("sm_mhz") if clocks else None
    line = {
        "metric": "swiglu_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": args.workload, "bs": bs, "sq": sq, "d_model": dm, "d_intermediate": di,
                   "parallelism": f"column-parallel d_intermediate x{world}" if world > 1 else "single GPU",
                   "timed_path": ("column_parallel_swiglu forward + backward (the package's multi-GPU API), "
                                  "x replicated, dX all-reduced " +
                                  ("by the library's own kernels over NVLink peer memory (PeerDxReducer)" if use_peer
                                   else "with NCCL beside the dW GEMM") if world > 1 else
                                  "the four launches of FusedSwiGLU forward + backward"),
                   "l2": "inputs larger than L2 (activations and weights exceed 126 MB); no flush",
                   "preheat_s": args.preheat, "preheat_steps": pre_steps,
                   "comm_sms_reserved_during_dw": parallel.comm_sms(world, group) if world > 1 and not use_peer else 0,
                   "dw_columns_beside_collective": dw_split["first"], "dw_columns_local": di_local,
                   "collective_ms_measured_alone": dw_split["collective_ms"],
                   "accumulate": "fp16 accumulator in forward and dW, fp32 in dX" if fast else "fp32",
                   "tile_options": {k: _lib.get_option(k) for k in ("cta_group", "nsub", "group_m")},
                   "producer_pacing": pacing,
                   "tile_note": "0 = chosen per launch; this workload gets CTA pairs, 256x512 tiles"},
        "frac_of_nominal_bf16_peak": value / (NOMINAL_BF16_TFLOPS * world),
        "frac_of_measured_sustained": value / (peaks["bf16_tflops_sustained"] * world),
        "ms_x_sm_mhz": ms_per_step * sm_mhz if sm_mhz else None,
        "fwd_tokens_per_s": fwd_tokens_per_s,
        "gpu_launches": n_launches * world,
        "per_rank_ms": per_rank,
        "clocks": clocks,
        "parity": parity,
        "roofline": roofline,
        "e2e": e2e,
        "cpu_baseline": cpu_baseline,
        "gpu_library_bar": gpu_bar,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

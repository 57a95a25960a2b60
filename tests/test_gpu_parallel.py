"""Column-parallel mode on real GPUs.  Two ranks, one per GPU, against the unsharded
single-GPU result (NCCL and the library's own peer-memory reduction; skipped on a box
with fewer than two GPUs), and the kernels of the peer-memory reduction with the ranks
emulated on one GPU."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist

    sys.path.insert(0, str(REPO))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from fused_swiglu import FusedSwiGLU
        from fusedswiglu_b200 import _lib, parallel

        gen = torch.Generator(device="cuda").manual_seed(0)  # same seed -> same tensors on every rank
        bs, sq, dm, di = 2, 512, 1024, 3072
        mk = lambda *s: torch.randn(*s, device="cuda", dtype=torch.bfloat16, generator=gen)
        x0, wg0, wu0, dout = mk(bs, sq, dm), mk(dm, di) / dm ** 0.5, mk(dm, di) / dm ** 0.5, mk(bs, sq, di)
        lo, hi = parallel.shard_bounds(di, rank, world)

        x = x0.clone().requires_grad_(True)
        wg = parallel.shard_columns(wg0, rank, world).requires_grad_(True)
        wu = parallel.shard_columns(wu0, rank, world).requires_grad_(True)
        out = parallel.column_parallel_swiglu(x, wg, wu)
        out.backward(dout[..., lo:hi].contiguous())
        out_full = parallel.unshard_columns(out.detach())

        xr = x0.clone().requires_grad_(True)
        wgr, wur = wg0.clone().requires_grad_(True), wu0.clone().requires_grad_(True)
        ref = FusedSwiGLU.apply(xr, wgr, wur)
        ref.backward(dout)
        torch.cuda.synchronize()

        def rel(a, b):
            return (torch.linalg.norm(a.float() - b.float()) / torch.linalg.norm(b.float())).item()

        # tokens sharded at the boundary too: all-gather of x, reduce-scatter of dX
        b0, b1 = rank * bs // world, (rank + 1) * bs // world
        xs_ = x0[b0:b1].clone().requires_grad_(True)
        wg2 = parallel.shard_columns(wg0, rank, world).requires_grad_(True)
        wu2 = parallel.shard_columns(wu0, rank, world).requires_grad_(True)
        out2 = parallel.column_parallel_swiglu(xs_, wg2, wu2, row_sharded=True)
        out2.backward(dout[..., lo:hi].contiguous())
        torch.cuda.synchronize()
        row_sharded = {
            "out_equal": bool(torch.equal(out2.detach(), out.detach())),
            "dwg_equal": bool(torch.equal(wg2.grad, wg.grad)),
            "dwu_equal": bool(torch.equal(wu2.grad, wu.grad)),
            "dx_shape_ok": tuple(xs_.grad.shape) == (bs // world, sq, dm),
            "dx_rel": rel(xs_.grad, xr.grad[b0:b1]),
        }

        # the same two modes with the dX collective done by the library's own kernels over
        # NVLink peer memory (three steps: both buffer sets and their reuse are exercised)
        reducers = {mode: parallel.PeerDxReducer(bs * sq, dm, torch.bfloat16, torch.device("cuda", rank), scatter=mode)
                    for mode in ("epilogue", "copy")}
        peer = {}
        for step in range(6):
            reducer = reducers["epilogue" if step < 3 else "copy"]
            x3 = x0.clone().requires_grad_(True)
            wg3 = parallel.shard_columns(wg0, rank, world).requires_grad_(True)
            wu3 = parallel.shard_columns(wu0, rank, world).requires_grad_(True)
            o3 = parallel.column_parallel_swiglu(x3, wg3, wu3, reducer=reducer)
            o3.backward(dout[..., lo:hi].contiguous())
            x4 = x0[b0:b1].clone().requires_grad_(True)
            wg4 = parallel.shard_columns(wg0, rank, world).requires_grad_(True)
            wu4 = parallel.shard_columns(wu0, rank, world).requires_grad_(True)
            o4 = parallel.column_parallel_swiglu(x4, wg4, wu4, row_sharded=True, reducer=reducer)
            o4.backward(dout[..., lo:hi].contiguous())
            torch.cuda.synchronize()
            peer[step] = {
                "dx_rel": rel(x3.grad, xr.grad), "dx_rows_rel": rel(x4.grad, xr.grad[b0:b1]),
                "dx_rows_equal_full": bool(torch.equal(x4.grad, x3.grad[b0:b1])),
                "dw_equal": bool(torch.equal(wg3.grad, wg.grad) and torch.equal(wu3.grad, wu.grad)
                                 and torch.equal(wg4.grad, wg.grad) and torch.equal(wu4.grad, wu.grad)),
            }
        # every rank holds the same reduced dX
        gathered = [torch.empty_like(x3.grad) for _ in range(world)]
        dist.all_gather(gathered, x3.grad.contiguous())
        peer["same_on_all_ranks"] = all(bool(torch.equal(t, gathered[0])) for t in gathered)

        # whole MLP block, tensor parallel vs single GPU
        from fusedswiglu_b200.mlp import FusedSwiGLUMLP

        wd0 = mk(di, dm) / di ** 0.5
        dy = mk(bs, sq, dm)
        xm = x0.clone().requires_grad_(True)
        wgm = parallel.shard_columns(wg0, rank, world).requires_grad_(True)
        wum = parallel.shard_columns(wu0, rank, world).requires_grad_(True)
        wdm = parallel.shard_rows(wd0, rank, world).requires_grad_(True)
        ym = parallel.TensorParallelSwiGLUMLP.apply(xm, wgm, wum, wdm)
        ym.backward(dy)
        xs = x0.clone().requires_grad_(True)
        wgs, wus, wds = (t.clone().requires_grad_(True) for t in (wg0, wu0, wd0))
        ys = FusedSwiGLUMLP.apply(xs, wgs, wus, wds)
        ys.backward(dy)
        torch.cuda.synchronize()
        mlp = {"y": rel(ym, ys), "dx": rel(xm.grad, xs.grad), "dwg": rel(wgm.grad, wgs.grad[:, lo:hi]),
               "dwu": rel(wum.grad, wus.grad[:, lo:hi]), "dwd": rel(wdm.grad, wds.grad[lo:hi])}

        q.put((rank, {
            "mlp": mlp,
            "row_sharded": row_sharded,
            "peer": peer,
            "out_equal": bool(torch.equal(out_full, ref.detach())),
            "dwg_equal": bool(torch.equal(wg.grad, wgr.grad[:, lo:hi])),
            "dwu_equal": bool(torch.equal(wu.grad, wur.grad[:, lo:hi])),
            "dx_rel": rel(x.grad, xr.grad),
            "status": _lib.device_status(),
        }))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_column_parallel_matches_single_gpu():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, r in results:
        # forward and dW shards are the same arithmetic as the unsharded run
        assert r["out_equal"] and r["dwg_equal"] and r["dwu_equal"], (rank, r)
        # dX: each rank rounds its partial sum to bf16 before the all-reduce
        assert r["dx_rel"] < 1e-2, (rank, r)
        assert r["status"] == 0
        rs = r["row_sharded"]
        assert rs["out_equal"] and rs["dwg_equal"] and rs["dwu_equal"] and rs["dx_shape_ok"], (rank, rs)
        assert rs["dx_rel"] < 1e-2, (rank, rs)
        for step in range(6):  # steps 0-2: partial sums stored by the GEMM epilogue, 3-5: by copy engines
            pr = r["peer"][step]
            assert pr["dx_rel"] < 1e-2 and pr["dx_rows_rel"] < 1e-2, (rank, step, pr)
            assert pr["dx_rows_equal_full"] and pr["dw_equal"], (rank, step, pr)
        assert r["peer"]["same_on_all_ranks"], rank
        # tensor-parallel MLP: partial sums are rounded per rank before the all-reduce
        for k, v in r["mlp"].items():
            assert v < 1e-2, (rank, k, r["mlp"])


def test_dx_scatter_and_reduction_with_the_ranks_emulated_on_one_gpu():
    """The kernels of the peer-memory dX reduction on ONE GPU: four 'ranks' with their own
    operands take turns on the device, every rank's receive buffer is local memory.  The
    scattering GEMM must put each rank's partial rows exactly where the owner expects
    them (tile order rotated per rank), and the reduction must give the fp32 sum of the
    slices in rank order, rounded once.  The flags are set from the host beforehand, so no
    kernel waits for another one."""
    import ctypes

    from fusedswiglu_b200 import _launch, _lib

    world, T, dm, di = 4, 2048, 512, 1024
    rows = T // world
    gen = torch.Generator(device="cuda").manual_seed(5)
    mk = lambda *s: torch.randn(*s, device="cuda", dtype=torch.bfloat16, generator=gen)
    ops = [(mk(T, di), mk(T, di), mk(dm, di) / di ** 0.5, mk(dm, di) / di ** 0.5) for _ in range(world)]
    recv = [torch.full((world, rows, dm), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    ptrs = [r.data_ptr() for r in recv]
    partial = []
    for r, (dg, du, wg, wu) in enumerate(ops):
        _launch.grad_input_scatter(dg, du, wg, wu, ptrs, world, r)
        partial.append(_launch.grad_input(dg, du, wg, wu, split_k=False))
    torch.cuda.synchronize()
    for owner in range(world):
        for src in range(world):
            assert torch.equal(recv[owner][src], partial[src][owner * rows:(owner + 1) * rows]), (owner, src)
    seq = 7
    flags = [torch.full((world,), seq, device="cuda", dtype=torch.int32) for _ in range(world)]
    fptrs = [f.data_ptr() for f in flags]
    for r in range(world):
        want = torch.zeros(rows, dm, device="cuda", dtype=torch.float32)
        for s in range(world):
            want += partial[s][r * rows:(r + 1) * rows].float()
        out = torch.full((rows, dm), float("nan"), device="cuda", dtype=torch.bfloat16)
        _launch.reduce_dx_slices(ptrs[r], fptrs, fptrs[r], world, r, seq, out)
        # the own slice read in place instead of from the receive buffer
        out2 = torch.empty_like(out)
        recv[r][r].fill_(float("nan"))
        _launch.reduce_dx_slices(ptrs[r], fptrs, fptrs[r], world, r, seq, out2,
                                 own_slice=partial[r][r * rows:(r + 1) * rows])
        torch.cuda.synchronize()
        assert torch.equal(out, want.to(torch.bfloat16)) and torch.equal(out2, out), r
    assert _lib.device_status() == 0


def test_a_reduction_whose_peers_never_signal_gives_up_and_reports_it():
    """No peer ever writes the flags: the reduction's time-limited wait runs out, the kernel
    records a status code, writes nothing and returns; the context stays usable.  (The wait
    is made to run out by a flag that nothing sets - no fault, no trap, no endless loop.)"""
    from fusedswiglu_b200 import _launch, _lib

    world, rows, dm = 2, 64, 64
    recv = torch.ones(world, rows, dm, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros(world, device="cuda", dtype=torch.int32)  # stay 0; the step number is 1
    out = torch.full((rows, dm), 5.0, device="cuda", dtype=torch.bfloat16)
    assert _lib.device_status() == 0
    old = _lib.get_option("wait_limit_ms")
    _lib.set_option("wait_limit_ms", 50)
    try:
        # this rank's own signal goes to word [1] of a scratch array, so word [1] of `flags` stays 0 too
        scratch = torch.zeros(world, device="cuda", dtype=torch.int32)
        _launch.reduce_dx_slices(recv.data_ptr(), [scratch.data_ptr(), scratch.data_ptr()], flags.data_ptr(),
                                 world, 1, 1, out)
        _launch.wait_flags(flags.data_ptr(), world, 1, out)
        torch.cuda.synchronize()
        status = _lib.load().fsw_status()
    finally:
        _lib.set_option("wait_limit_ms", old)
    assert status != 0 and (status & 0x7F) == 5, status       # WAIT_PEER_PARTIALS
    assert "bounded wait" in _lib.last_error()
    assert bool((out == 5.0).all())                           # nothing was written
    assert _lib.device_status() == 0                          # reading the status cleared it
    flags.fill_(1)
    _launch.reduce_dx_slices(recv.data_ptr(), [scratch.data_ptr(), scratch.data_ptr()], flags.data_ptr(),
                             world, 1, 1, out)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0 and bool((out == 2.0).all())

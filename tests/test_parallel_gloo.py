"""Host logic of the column-parallel mode on CPU: two gloo ranks, with the GPU
launches replaced by a CPU stand-in built from the oracle's torch formula.  The
stand-in is test scaffolding; the product's backend is CUDA-only."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parent.parent


class OracleBackend:
    """CPU stand-in with the launchers' signatures, fp32 math on 16-bit tensors."""

    @staticmethod
    def forward(x2d, wg, wu, *, fast_accum=False, save_activations=True):
        g = (x2d.float() @ wg.float()).to(x2d.dtype)
        u = (x2d.float() @ wu.float()).to(x2d.dtype)
        out = (torch.nn.functional.silu(g.float()) * u.float()).to(x2d.dtype)
        return out, g, u

    @staticmethod
    def gate_grad(dout, g, u):
        gf = g.float()
        s = torch.sigmoid(gf)
        du = (dout.float() * gf * s).to(dout.dtype)
        dg = (dout.float() * u.float() * (s + gf * s * (1 - s))).to(dout.dtype)
        return dg, du

    @staticmethod
    def grad_input(dg, du, wg, wu):
        return (dg.float() @ wg.float().T + du.float() @ wu.float().T).to(dg.dtype)

    @staticmethod
    def grad_weights(x2d, dg, du, *, fast_accum=False):
        return (x2d.float().T @ dg.float()).to(x2d.dtype), (x2d.float().T @ du.float()).to(x2d.dtype)

    @staticmethod
    def gemm(a, b, *, trans_a=False, trans_b=False, fast_accum=False):
        a32 = a.float().T if trans_a else a.float()
        b32 = b.float().T if trans_b else b.float()
        return (a32 @ b32).to(a.dtype)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, str(REPO))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fusedswiglu_b200 import parallel
        from oracle import swiglu_oracle as orc

        torch.manual_seed(0)
        bs, sq, dm, di = 2, 32, 64, 128
        x = torch.randn(bs, sq, dm).bfloat16().requires_grad_(True)
        wg = (torch.randn(dm, di) / dm ** 0.5).bfloat16()
        wu = (torch.randn(dm, di) / dm ** 0.5).bfloat16()
        dout = torch.randn(bs, sq, di).bfloat16()
        lo, hi = parallel.shard_bounds(di, rank, world)
        wg_s = parallel.shard_columns(wg, rank, world).requires_grad_(True)
        wu_s = parallel.shard_columns(wu, rank, world).requires_grad_(True)
        out_s = parallel.ColumnParallelSwiGLU.apply(x, wg_s, wu_s, None, False, OracleBackend)
        out_s.backward(dout[..., lo:hi].contiguous())
        out_full = parallel.unshard_columns(out_s.detach())

        xr = x.detach().clone().requires_grad_(True)
        wgr = wg.clone().requires_grad_(True)
        wur = wu.clone().requires_grad_(True)
        ref = orc.swiglu_ref_torch(xr, wgr, wur)
        ref.backward(dout)

        def rel(a, b):
            return (torch.linalg.norm(a.float() - b.float()) / torch.linalg.norm(b.float())).item()

        errs = {
            "out": rel(out_full, ref),
            "dx": rel(x.grad, xr.grad),
            "dwg": rel(wg_s.grad, wgr.grad[:, lo:hi]),
            "dwu": rel(wu_s.grad, wur.grad[:, lo:hi]),
        }
        # every rank must hold the same reduced dX
        gathered = [torch.empty_like(x.grad) for _ in range(world)]
        dist.all_gather(gathered, x.grad)
        errs["dx_equal_across_ranks"] = float(max((g.float() - gathered[0].float()).abs().max() for g in gathered))
        q.put((rank, errs))
    finally:
        dist.destroy_process_group()


def test_two_rank_column_parallel_matches_unsharded_reference():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in results:
        assert errs["dx_equal_across_ranks"] == 0.0, (rank, errs)
        for k in ("out", "dx", "dwg", "dwu"):
            assert errs[k] < 1e-2, (rank, k, errs)


def _mlp_worker(rank, world, port, q):
    sys.path.insert(0, str(REPO))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fusedswiglu_b200 import parallel

        torch.manual_seed(1)
        bs, sq, dm, di = 2, 16, 64, 128
        x = torch.randn(bs, sq, dm).bfloat16().requires_grad_(True)
        wg = (torch.randn(dm, di) / dm ** 0.5).bfloat16()
        wu = (torch.randn(dm, di) / dm ** 0.5).bfloat16()
        wd = (torch.randn(di, dm) / di ** 0.5).bfloat16()
        dy = torch.randn(bs, sq, dm).bfloat16()
        lo, hi = parallel.shard_bounds(di, rank, world)
        wg_s = parallel.shard_columns(wg, rank, world).requires_grad_(True)
        wu_s = parallel.shard_columns(wu, rank, world).requires_grad_(True)
        wd_s = parallel.shard_rows(wd, rank, world).requires_grad_(True)
        y = parallel.TensorParallelSwiGLUMLP.apply(x, wg_s, wu_s, wd_s, None, OracleBackend)
        y.backward(dy)

        xr = x.detach().clone().requires_grad_(True)
        wgr, wur, wdr = (t.clone().requires_grad_(True) for t in (wg, wu, wd))
        ref = (torch.nn.functional.silu(xr @ wgr) * (xr @ wur)) @ wdr
        ref.backward(dy)

        def rel(a, b):
            return (torch.linalg.norm(a.float() - b.float()) / torch.linalg.norm(b.float())).item()

        q.put((rank, {"y": rel(y, ref), "dx": rel(x.grad, xr.grad), "dwg": rel(wg_s.grad, wgr.grad[:, lo:hi]),
                      "dwu": rel(wu_s.grad, wur.grad[:, lo:hi]), "dwd": rel(wd_s.grad, wdr.grad[lo:hi])}))
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_mlp_matches_unsharded_reference():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_mlp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in results:
        for k, v in errs.items():
            assert v < 2e-2, (rank, k, errs)


def test_shard_bounds_and_errors():
    from fusedswiglu_b200 import parallel

    assert parallel.shard_bounds(14336, 3, 8) == (5376, 7168)
    assert [parallel.shard_bounds(28672, r, 4)[0] for r in range(4)] == [0, 7168, 14336, 21504]
    with pytest.raises(ValueError, match="not divisible"):
        parallel.shard_bounds(100, 0, 3)
    with pytest.raises(ValueError, match="multiple of 8"):
        parallel.shard_bounds(72, 0, 2)  # 36 columns per rank
    with pytest.raises(ValueError, match="bad rank"):
        parallel.shard_bounds(64, 2, 2)
    w = torch.arange(4 * 32).view(4, 32)
    s = parallel.shard_columns(w, 1, 2)
    assert s.is_contiguous() and torch.equal(s, w[:, 16:])


def _absent_rank_worker(rank, world, port, q):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        if rank == 0:
            try:
                dist.all_reduce(torch.ones(4))
                q.put("completed")
            except Exception as e:  # the collective must end with an error, not hang
                q.put("error:" + type(e).__name__)
        else:
            q.put("absent")  # this rank never joins the collective
            import time

            time.sleep(8)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_plan_of_the_dw_split_beside_the_all_reduce():
    """The column count that runs beside the collective is a whole number of tiles,
    grows with the collective's size relative to the GEMM, and covers the whole GEMM
    when the collective is the longer of the two."""
    from fusedswiglu_b200.parallel import plan_dw_split, DW_SPLIT_ALIGN

    assert plan_dw_split(32768, 4096, 14336, 1, 148, 16) == 0          # no collective
    assert plan_dw_split(32768, 4096, 7168, 2, 148, 0) == 0            # nothing reserved
    for T, dm, di, world, reserve in [(32768, 4096, 7168, 2, 16), (65536, 8192, 7168, 4, 32),
                                      (65536, 8192, 14336, 2, 16)]:
        c = plan_dw_split(T, dm, di, world, 148, reserve)
        assert 0 < c < di and c % DW_SPLIT_ALIGN == 0, (T, dm, di, world, c)
    # 8 ranks: the local GEMM is shorter than the all-reduce of the full dX
    assert plan_dw_split(32768, 4096, 1792, 8, 148, 32) == 1792
    # tiny problems are dominated by the collective's fixed cost
    assert plan_dw_split(128, 512, 768, 2, 148, 16) == 768
    # the same collective beside a GEMM twice as long covers a smaller share of it
    assert plan_dw_split(65536, 8192, 14336, 2, 148, 16) / 14336 < plan_dw_split(65536, 8192, 7168, 2, 148, 16) / 7168


def test_dw_beside_collective_call_sequence(monkeypatch):
    """Host logic of the dW launch beside the collective, with the library and the
    launchers replaced by recorders (no GPU): the SM cap is an argument of the first
    launch only (no process-wide option is touched), the stream waits for the
    collective before the rest, and the rest runs uncapped."""
    import torch
    from fusedswiglu_b200 import parallel

    log = []

    class FakeLib:
        @staticmethod
        def get_option(name):
            return {"sm_count": 148}[name]

        @staticmethod
        def set_option(name, value):  # must not be called
            raise AssertionError(f"process-wide option {name} was set")

    class FakeLaunch:
        @staticmethod
        def grad_weights(x2d, dg, du, *, fast_accum=False, out_gate=None, out_up=None, columns=None, max_sms=0):
            log.append(("dw", columns, max_sms, out_gate is not None))
            return (out_gate if out_gate is not None else "dwg"), (out_up if out_up is not None else "dwu")

    class Work:
        def wait(self):
            log.append(("wait",))

    monkeypatch.setattr(parallel, "_lib", FakeLib)
    monkeypatch.setattr(parallel, "_launch", FakeLaunch)
    x2d, dg = torch.empty(65536, 8192, dtype=torch.bfloat16, device="meta"), torch.empty(65536, 7168, dtype=torch.bfloat16, device="meta")
    first = parallel.plan_dw_split(65536, 8192, 7168, 4, 148, 32)
    out = parallel._CudaBackend.grad_weights_beside_collective(x2d, dg, dg, world_size=4, work=Work())
    assert out == ("dwg", "dwu")
    assert log == [("dw", (0, first), 116, False), ("wait",), ("dw", (first, 7168 - first), 0, True)]
    # a reduce-scatter moves half the bytes of an all-reduce: a smaller first part
    log.clear()
    first_rs = parallel.plan_dw_split(65536, 8192, 7168, 4, 148, 32, collective="reduce_scatter")
    assert 0 < first_rs < first
    parallel._CudaBackend.grad_weights_beside_collective(x2d, dg, dg, world_size=4, work=Work(),
                                                         collective="reduce_scatter")
    assert log == [("dw", (0, first_rs), 116, False), ("wait",), ("dw", (first_rs, 7168 - first_rs), 0, True)]
    # the collective outlasts the GEMM (8 ranks, 8B shape): one launch, all of it on the reduced SM count
    log.clear()
    x2d, dg = torch.empty(32768, 4096, dtype=torch.bfloat16, device="meta"), torch.empty(32768, 1792, dtype=torch.bfloat16, device="meta")
    parallel._CudaBackend.grad_weights_beside_collective(x2d, dg, dg, world_size=8, work=Work())
    assert log == [("dw", None, 116, False)]


def _row_sharded_worker(rank, world, port, q):
    sys.path.insert(0, str(REPO))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fusedswiglu_b200 import parallel
        from oracle import swiglu_oracle as orc

        torch.manual_seed(0)
        bs, sq, dm, di = 4, 16, 64, 128
        x = torch.randn(bs, sq, dm).bfloat16()
        wg = (torch.randn(dm, di) / dm ** 0.5).bfloat16()
        wu = (torch.randn(dm, di) / dm ** 0.5).bfloat16()
        dout = torch.randn(bs, sq, di).bfloat16()
        lo, hi = parallel.shard_bounds(di, rank, world)
        b0, b1 = rank * bs // world, (rank + 1) * bs // world
        x_mine = x[b0:b1].clone().requires_grad_(True)
        wg_s = parallel.shard_columns(wg, rank, world).requires_grad_(True)
        wu_s = parallel.shard_columns(wu, rank, world).requires_grad_(True)
        out_s = parallel.column_parallel_swiglu(x_mine, wg_s, wu_s, row_sharded=True, backend=OracleBackend)
        assert out_s.shape == (bs, sq, hi - lo)
        out_s.backward(dout[..., lo:hi].contiguous())
        assert x_mine.grad.shape == (bs // world, sq, dm)
        out_full = parallel.unshard_columns(out_s.detach())

        xr = x.clone().requires_grad_(True)
        wgr = wg.clone().requires_grad_(True)
        wur = wu.clone().requires_grad_(True)
        ref = orc.swiglu_ref_torch(xr, wgr, wur)
        ref.backward(dout)

        def rel(a, b):
            return (torch.linalg.norm(a.float() - b.float()) / torch.linalg.norm(b.float())).item()

        q.put((rank, {"out": rel(out_full, ref), "dx": rel(x_mine.grad, xr.grad[b0:b1]),
                      "dwg": rel(wg_s.grad, wgr.grad[:, lo:hi]), "dwu": rel(wu_s.grad, wur.grad[:, lo:hi])}))
    finally:
        dist.destroy_process_group()


def test_two_rank_row_sharded_mode_matches_unsharded_reference():
    """Tokens sharded at the boundary: all-gather of x in forward, reduce-scatter of
    dX in backward; every rank gets the gradient of its own rows."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_row_sharded_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in results:
        for k, v in errs.items():
            assert v < 1e-2, (rank, k, errs)


def test_rank_that_never_joins_ends_the_collective_with_an_error():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_absent_rank_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    msgs = sorted(q.get(timeout=60) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
    assert msgs[0] == "absent" and msgs[1].startswith("error:"), msgs


def test_peer_reducer_buffer_sets_alternate_and_never_overlap():
    """Host arithmetic of PeerDxReducer: consecutive steps use different buffer sets,
    a set's receive slices, row blocks and flag words stay inside the set, and the two
    kinds of flag words of the two sets are four disjoint groups of `world` words."""
    from fusedswiglu_b200.parallel import PeerDxReducer

    T, dm, esize = 4096, 512, 2
    for world in (2, 4, 8):
        rows = T // world
        words = set()
        for seq in (1, 2, 3, 4):
            lays = [PeerDxReducer.layout(seq, world, r, T, dm, esize) for r in range(world)]
            s = lays[0]["set"]
            assert s == seq & 1 and all(l["set"] == s for l in lays)
            assert lays[0]["recv_byte_offset"] == s * T * dm * esize
            # slice [source][rows][dm] of one set is exactly T*dm elements: sets do not overlap
            assert world * rows * dm * esize == T * dm * esize
            blocks = [l["my_block_elem_offset"] for l in lays]
            assert blocks == [s * T * dm + r * rows * dm for r in range(world)]
            assert blocks[-1] + rows * dm == (s + 1) * T * dm
            for kind in (0, 1):
                first = lays[0]["flag_word"][kind]
                assert 0 <= first and first + world <= 4 * world
                if seq <= 2:
                    group = set(range(first, first + world))
                    assert not (group & words)
                    words |= group
        assert len(words) == 4 * world
        assert PeerDxReducer.layout(1, world, 0, T, dm, esize)["set"] != PeerDxReducer.layout(2, world, 0, T, dm, esize)["set"]
        assert PeerDxReducer.layout(1, world, 0, T, dm, esize) == PeerDxReducer.layout(3, world, 0, T, dm, esize)


def test_dw_columns_queued_before_the_peer_reduction():
    """Host planning of PeerDxReducer: how the local dW GEMM is cut around the reduction.
    Row-sharded mode has no gather to cover, so all of dW comes first; in replicated-x mode
    the part after the reduction lasts about as long as the copy-engine gather and is a
    whole number of tiles; with copy-engine scatter and a GEMM too short for two rounds of
    copies each round gets half."""
    from types import SimpleNamespace

    from fusedswiglu_b200.parallel import DW_SPLIT_ALIGN, PeerDxReducer

    def reducer(world, T, dm, mode="epilogue"):
        return SimpleNamespace(world=world, T=T, dm=dm, rows=T // world, esize=2, scatter_mode=mode)

    plan = PeerDxReducer.columns_before_reduction
    for world, di_local in ((2, 7168), (4, 3584), (8, 1792)):
        r = reducer(world, 32768, 4096)
        assert plan(r, di_local, True) == di_local
        first = plan(r, di_local, False)
        assert 0 <= first < di_local and (di_local - first) % DW_SPLIT_ALIGN == 0
    # the longer the GEMM relative to the gather, the larger the share that comes first
    assert plan(reducer(2, 32768, 4096), 7168, False) / 7168 > plan(reducer(8, 32768, 4096), 1792, False) / 1792
    # copy-engine scatter, 8 ranks: the GEMM (0.7 ms) is shorter than two rounds of copies
    half = plan(reducer(8, 32768, 4096, "copy"), 1792, False)
    assert half == (1792 // 2) // DW_SPLIT_ALIGN * DW_SPLIT_ALIGN

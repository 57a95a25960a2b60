"""Column-parallel SwiGLU across the GPUs of one node.

``d_intermediate`` is split evenly over the ranks of a ``torch.distributed``
process group (one process per GPU).  Rank r holds columns
``[r*di/P, (r+1)*di/P)`` of W_gate and W_up and every rank holds the whole x, so

  * forward is purely local: rank r produces its slice ``out[..., r*di/P:(r+1)*di/P]``;
  * backward is local for dW_gate/dW_up (their column slices) and produces a
    PARTIAL dX on every rank; the one collective on the path is the all-reduce
    (sum) of dX.  It is started as soon as the dX GEMM has been queued and runs on
    NCCL's stream while the dW GEMM - which does not depend on dX - computes; the
    backward joins the two before it returns.

With ``row_sharded=True`` the tokens are sharded as well at the boundary of the
call (sequence parallel): rank r passes rows ``[r*T/P, (r+1)*T/P)`` of x, the
forward all-gathers them over NVLink, and the backward ends in a reduce-scatter of
dX, so each rank gets back the gradient of its own rows only.  Per-rank host
traffic and the collective's wire bytes then shrink with the number of ranks
(``(P-1)/P`` of dX crosses NVLink instead of ``2(P-1)/P``).

The reference (fattorib/fusedswiglu) has no multi-GPU mode; this follows the
standard tensor-parallel MLP split and keeps the single-GPU numerics per shard.
"""
from __future__ import annotations

import contextlib
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist
from torch.autograd import Function

from . import _launch, _lib

# SMs left free for the collective's kernel while the dW GEMM runs.  The GEMMs are
# persistent and would otherwise occupy every SM, so that NCCL's kernel could not
# start before they finish and the collective would not overlap anything.  NCCL's
# kernels only make progress once ALL of their CTAs are resident, so the number of
# free SMs must cover the CTAs NCCL launches: a group made by new_collective_group()
# caps them (NCCL config max_ctas) and exactly that many SMs are reserved; for any
# other group 16 SMs (2 ranks) or 32 (more; NCCL's default channel count there) are.
# FSW_COMM_SMS overrides; 0 disables the cap.
_COMM_SMS_ENV = os.environ.get("FSW_COMM_SMS")
_GROUP_MAX_CTAS = {}  # process group -> CTA cap it was created with
DEFAULT_COLLECTIVE_CTAS = 16


def new_collective_group(ranks=None, max_ctas: int = DEFAULT_COLLECTIVE_CTAS, **kwargs):
    """A process group for the dX collective whose NCCL kernels launch at most
    ``max_ctas`` CTAs, so that they fit into the SMs the dW GEMM leaves free beside
    them (pass it as ``group=``).  On a non-NCCL backend this is a plain new_group."""
    if dist.get_backend() != "nccl":
        return dist.new_group(ranks, **kwargs)
    opts = dist.ProcessGroupNCCL.Options()
    opts.config.max_ctas = int(max_ctas)
    opts.config.min_ctas = min(int(max_ctas), 4)
    group = dist.new_group(ranks, pg_options=opts, **kwargs)
    _GROUP_MAX_CTAS[group] = int(max_ctas)
    return group


def comm_sms(world_size: int, group=None) -> int:
    if _COMM_SMS_ENV is not None:
        return int(_COMM_SMS_ENV)
    if group is not None and group in _GROUP_MAX_CTAS:
        return _GROUP_MAX_CTAS[group]
    return 16 if world_size <= 2 else 32


# Duration of the dX collective, measured once per (group, message, kind) on the
# first backward that needs it (two timed runs on a scratch tensor, synchronously -
# like an autotuner's first call) and used from then on to size the part of the dW
# GEMM that runs beside it.  Without a CUDA tensor (CPU tests) the planning figures
# below are used instead.
_COLLECTIVE_SECONDS = {}


def collective_seconds(dx: torch.Tensor, group, collective: str) -> Optional[float]:
    if not dx.is_cuda:
        return None
    key = (group, dx.numel() * dx.element_size(), collective)
    if key not in _COLLECTIVE_SECONDS:
        world = dist.get_world_size(group)
        src = torch.zeros_like(dx)
        dst = torch.empty((dx.shape[0] // world, dx.shape[1]), device=dx.device, dtype=dx.dtype) \
            if collective == "reduce_scatter" else None
        best = None
        for i in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if dst is not None:
                dist.reduce_scatter_tensor(dst, src, group=group)
            else:
                dist.all_reduce(src, group=group)
            e1.record()
            e1.synchronize()
            if i > 0:
                t = e0.elapsed_time(e1) * 1e-3
                best = t if best is None else min(best, t)
        _COLLECTIVE_SECONDS[key] = best
    return _COLLECTIVE_SECONDS[key]


# Planning figures used when the collective has not been measured (see
# collective_seconds): the bus bandwidth NCCL reaches through NVSwitch while confined
# to a few SMs beside a GEMM, its fixed cost, and the sustained rate of the GEMM on
# the full GPU.
ALLREDUCE_BUS_BYTES_PER_S = {2: 215e9, 4: 225e9, 8: 490e9}
ALLREDUCE_BUS_BYTES_PER_S_OTHER = 225e9
ALLREDUCE_FIXED_S = 40e-6
GEMM_SUSTAINED_FLOPS = 1.35e15
DW_SPLIT_ALIGN = 256  # columns per dW tile
GATHER_BYTES_PER_S = 650e9  # copy-engine peer copies into one GPU over NVLink (measured: ~700 GB/s per pair)


def plan_dw_split(T: int, dm: int, di_local: int, world_size: int, sm_count: int, reserve: int,
                  elem_bytes: int = 2, collective: str = "all_reduce",
                  measured_seconds: Optional[float] = None) -> int:
    """Columns of the local dW GEMM to run on ``sm_count - reserve`` SMs beside the
    collective on dX (T x dm elements; ``"all_reduce"`` or ``"reduce_scatter"``, which
    moves half the bytes); the remaining columns run afterwards on all SMs.  The
    first part is sized to last 1.1x the estimated collective time; returns
    ``di_local`` when the whole GEMM is needed to cover it.  ``measured_seconds`` is the
    collective's measured duration, if known; otherwise it is estimated."""
    if world_size <= 1 or reserve <= 0:
        return 0
    if measured_seconds is not None:
        t_ar = measured_seconds
    else:
        bus = ALLREDUCE_BUS_BYTES_PER_S.get(world_size, ALLREDUCE_BUS_BYTES_PER_S_OTHER)
        passes = 2.0 if collective == "all_reduce" else 1.0
        t_ar = passes * (world_size - 1) / world_size * T * dm * elem_bytes / bus
        t_ar += ALLREDUCE_FIXED_S
    rate = GEMM_SUSTAINED_FLOPS * max(1, sm_count - reserve) / sm_count
    t_dw = 4.0 * T * dm * di_local / rate
    cols = int(di_local * min(1.0, 1.1 * t_ar / t_dw))
    cols = -(-cols // DW_SPLIT_ALIGN) * DW_SPLIT_ALIGN
    # a tail of less than two tiles is not worth a launch of its own
    if cols + 2 * DW_SPLIT_ALIGN > di_local:
        return di_local
    return cols


def shard_bounds(d_intermediate: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Column range of `rank`; d_intermediate must split into equal 8-aligned parts."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if d_intermediate % world_size != 0:
        raise ValueError(f"d_intermediate={d_intermediate} is not divisible by world_size={world_size}")
    per = d_intermediate // world_size
    if per % 8 != 0:
        raise ValueError(
            f"shard width {per} (= {d_intermediate}/{world_size}) must be a multiple of 8 (16-byte rows)"
        )
    return rank * per, (rank + 1) * per


def shard_columns(w: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """Contiguous copy of this rank's column slice of a (d_model, d_intermediate) weight."""
    lo, hi = shard_bounds(w.shape[1], rank, world_size)
    return w[:, lo:hi].contiguous()


def unshard_columns(shard: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather column slices (last dimension) back into the full tensor."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(shard) for _ in range(world)]
    dist.all_gather(parts, shard.contiguous(), group=group)
    return torch.cat(parts, dim=-1)


class _CudaBackend:
    """The product compute path: C-ABI launches on the current CUDA stream."""

    forward = staticmethod(_launch.forward)
    gate_grad = staticmethod(_launch.gate_grad)
    grad_input = staticmethod(_launch.grad_input)
    grad_weights = staticmethod(_launch.grad_weights)
    gemm = staticmethod(_launch.gemm)

    @staticmethod
    def grad_weights_beside_collective(x2d, dg, du, *, fast_accum=False, world_size=2, work=None,
                                       collective="all_reduce", group=None, collective_s=None):
        """dW GEMM while the collective on dX (``work``) is in flight.

        NCCL's kernel makes no progress until all of its CTAs are resident, so the
        columns of dW that overlap it run on all but comm_sms(world_size) SMs.  When
        the GEMM is longer than the collective, only a first column range sized to
        the collective's estimated duration runs that way; the current stream then
        waits for the collective and the remaining columns get the whole GPU."""
        reserve = comm_sms(world_size, group)
        if reserve <= 0:
            return _launch.grad_weights(x2d, dg, du, fast_accum=fast_accum)
        with torch.cuda.device(x2d.device) if x2d.is_cuda else contextlib.nullcontext():
            sms = _lib.get_option("sm_count")  # of the device the tensors live on
        T, dm = x2d.shape
        di = dg.shape[1]
        first = (plan_dw_split(T, dm, di, world_size, sms, reserve, x2d.element_size(), collective,
                               collective_s)
                 if work is not None else di)
        cap = max(2, sms - reserve)  # an argument of this one launch, not process-wide state
        if first >= di:
            return _launch.grad_weights(x2d, dg, du, fast_accum=fast_accum, max_sms=cap)
        dwg, dwu = _launch.grad_weights(x2d, dg, du, fast_accum=fast_accum, columns=(0, first), max_sms=cap)
        work.wait()  # stream-level: the rest starts when the collective's kernel has left the SMs
        return _launch.grad_weights(x2d, dg, du, fast_accum=fast_accum, out_gate=dwg, out_up=dwu,
                                    columns=(first, di - first))


class PeerDxReducer:
    """The dX collective done by this library's own kernels over NVLink peer memory
    instead of NCCL (pass as ``reducer=`` to column_parallel_swiglu).

    Every rank's dX GEMM stores its partial sums from its epilogue straight into the
    receive buffer of the rank that owns the rows (reduce-scatter, no extra pass over
    the partials and no SM taken from a GEMM); a short kernel then waits - with a time
    limit - for the peers' partials and adds the slices in fp32 in rank order, so the
    result is deterministic and rounded once.  For the replicated-x mode the reduced
    row blocks are then copied to every peer by plain device-to-device copies on a side
    stream (copy engines, no SMs) while the dW GEMM has the whole GPU, and a last
    time-limited wait confirms that the peers' blocks have landed.

    Buffers live in symmetric memory (torch.distributed._symmetric_memory: the same
    allocation on every rank, each mapped into every process); only plain loads, stores
    and copies touch peer memory.  Two sets alternate from step to step: a rank can be
    one step ahead of a peer, never two, because its reduction waits for every peer's
    signal of the same step.

    ``scatter="copy"`` is the variant without peer stores from the GEMM: the dX GEMM
    writes its partial sums locally at full speed and copy engines carry each row block
    to its owner (beside the first column range of the dW GEMM); reduction and gather are
    the same.  It moves the same bytes without any SM stalling on NVLink stores, but needs
    a dW GEMM long enough to cover two rounds of copies.

    In replicated-x mode the returned dX is a view of an internal buffer that the
    second-next call overwrites; pass ``own_output=True`` to get a private copy.
    Collective: construct it on all ranks of ``group`` at the same point."""

    def __init__(self, T: int, dm: int, dtype: torch.dtype, device, group=None, own_output: bool = False,
                 scatter: str = "epilogue"):
        if scatter not in ("epilogue", "copy"):
            raise ValueError("scatter must be 'epilogue' or 'copy'")
        self.scatter_mode = scatter
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer access only
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if not 2 <= self.world <= 8:
            raise ValueError(f"PeerDxReducer serves 2..8 ranks, got {self.world}")
        if T % self.world or (T // self.world) % 32:
            raise ValueError(f"T={T} must split into {self.world} equal parts of a multiple of 32 rows")
        self.T, self.dm, self.dtype, self.device = T, dm, dtype, torch.device(device)
        self.rows = T // self.world
        self.own_output = own_output
        self.seq = 0
        self.esize = torch.empty((), dtype=dtype).element_size()
        self.recv = symm_mem.empty(2 * T * dm, dtype=dtype, device=self.device)       # [set][source][rows][dm]
        self.full = symm_mem.empty(2 * T * dm, dtype=dtype, device=self.device)       # [set][T][dm]
        self.flags = symm_mem.empty(2 * 2 * self.world, dtype=torch.int32, device=self.device)  # [set][kind][rank]
        self.flags.zero_()
        self.h_recv = symm_mem.rendezvous(self.recv, self.group)
        self.h_full = symm_mem.rendezvous(self.full, self.group)
        self.h_flags = symm_mem.rendezvous(self.flags, self.group)
        self.side = torch.cuda.Stream(device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # every rank's flags are zero before anyone signals

    # ---- layout of the two buffer sets (host arithmetic; has a CPU test)
    @staticmethod
    def layout(seq: int, world: int, rank: int, T: int, dm: int, esize: int) -> dict:
        """Byte / element offsets used by step ``seq`` (1, 2, ...): which buffer set, where
        the set's receive slices start, where this rank's row block sits in the gathered
        dX, and the first flag word of the set's "partials arrived" (kind 0) and "row
        blocks gathered" (kind 1) arrays."""
        s = seq & 1
        rows = T // world
        return {
            "set": s,
            "recv_byte_offset": s * T * dm * esize,           # [set][source rank][rows][dm]
            "full_elem_offset": s * T * dm,                   # [set][T][dm]
            "my_block_elem_offset": s * T * dm + rank * rows * dm,
            "flag_word": {kind: (s * 2 + kind) * world for kind in (0, 1)},  # [set][kind][rank]
        }

    def _recv_ptrs(self, s):
        return [p + s * self.T * self.dm * self.esize for p in self.h_recv.buffer_ptrs]

    def _flag_ptrs(self, s, kind):
        return [p + ((s * 2 + kind) * self.world) * 4 for p in self.h_flags.buffer_ptrs]

    def scatter(self, dg, du, w_gate, w_up) -> None:
        """Queue this step's dX GEMM; its epilogue stores the partial sums into the
        owning ranks' receive buffers."""
        self.seq += 1
        self._lay = lay = self.layout(self.seq, self.world, self.rank, self.T, self.dm, self.esize)
        self._copied = None
        if self.scatter_mode == "epilogue":
            _launch.grad_input_scatter(dg, du, w_gate, w_up, self._recv_ptrs(lay["set"]), self.world, self.rank)
            return
        # copy engines carry the row blocks of the locally written partial dX to their owners
        rank, world, rows, dm = self.rank, self.world, self.rows, self.dm
        self._partial = partial = _launch.grad_input(dg, du, w_gate, w_up)
        done = torch.cuda.Event()
        done.record()
        with torch.cuda.stream(self.side):
            self.side.wait_event(done)
            off = lay["set"] * self.T * dm + rank * rows * dm  # slice [this rank] of the owner's buffer
            for r in [(rank + k) % world for k in range(1, world)]:  # the own block stays where it is
                self.h_recv.get_buffer(r, (rows, dm), self.dtype, off).copy_(partial[r * rows:(r + 1) * rows],
                                                                             non_blocking=True)
            self._copied = torch.cuda.Event()
            self._copied.record()

    def columns_before_reduction(self, di_local: int, row_sharded: bool) -> int:
        """How many columns of the local dW GEMM to queue between scatter() and reduce().

        The reduction waits for the slowest peer's dX GEMM; GEMM work queued before it
        absorbs that wait.  In replicated-x mode the rest of dW, queued after it, must
        still last as long as the gather of the row blocks (copy engines, about
        650 GB/s into each GPU), or the gather is left exposed."""
        if row_sharded:
            return di_local
        nbytes = (self.world - 1) * self.rows * self.dm * self.esize
        t_gather = 1.15 * (nbytes / GATHER_BYTES_PER_S + 30e-6)
        t_dw = 4.0 * self.T * self.dm * di_local / GEMM_SUSTAINED_FLOPS
        if self.scatter_mode == "copy" and 2 * t_gather >= t_dw:
            # two rounds of copies (to the owners, then the gather) and a GEMM too short to
            # cover both: give each round half of it
            return (di_local // 2) // DW_SPLIT_ALIGN * DW_SPLIT_ALIGN
        after = min(1.0, t_gather / t_dw) * di_local
        after = min(di_local, -(-int(after) // DW_SPLIT_ALIGN) * DW_SPLIT_ALIGN)
        return di_local - after

    def reduce(self, row_sharded: bool):
        """Queue the reduction of this step's partials (after scatter()).  Returns
        (dx, finish): call ``finish()`` after queueing the work that should overlap
        the gather; dx is valid on the current stream after it."""
        seq, rank, world, rows, dm, lay = self.seq, self.rank, self.world, self.rows, self.dm, self._lay
        s = lay["set"]
        if self._copied is not None:
            # the kernel below tells the peers that this rank's partials have arrived:
            # true only once the copies have
            torch.cuda.current_stream(self.device).wait_event(self._copied)
        if row_sharded:
            mine = torch.empty((rows, dm), device=self.device, dtype=self.dtype)
        else:
            full = self.full[lay["full_elem_offset"]:lay["full_elem_offset"] + self.T * dm].view(self.T, dm)
            mine = full[rank * rows:(rank + 1) * rows]
        own = self._partial[rank * rows:(rank + 1) * rows] if self._copied is not None else None
        _launch.reduce_dx_slices(self._recv_ptrs(s)[rank], self._flag_ptrs(s, 0), self._flag_ptrs(s, 0)[rank],
                                 world, rank, seq, mine, own_slice=own)
        if row_sharded:
            return mine, (lambda: mine)
        # gather: my reduced rows to every peer's copy of the full dX, then my step
        # number into their "gathered" flag word for me - device-to-device copies
        # queued on a side stream, ordered after the reduction
        done = torch.cuda.Event()
        done.record()
        with torch.cuda.stream(self.side):
            self.side.wait_event(done)
            off = lay["my_block_elem_offset"]
            # rank i sends to i+1, i+2, ...: at every moment the ranks write to different GPUs
            order = [(rank + k) % world for k in range(1, world)]
            for r in order:
                self.h_full.get_buffer(r, (rows, dm), self.dtype, off).copy_(mine, non_blocking=True)
            w0, w1 = lay["flag_word"][0] + rank, lay["flag_word"][1] + rank
            src = self.flags[w0:w0 + 1]  # my own "partials arrived" word: holds seq now
            for r in order + [rank]:
                self.h_flags.get_buffer(r, (1,), torch.int32, w1).copy_(src, non_blocking=True)

        def finish():
            _launch.wait_flags(self._flag_ptrs(s, 1)[rank], world, seq, full)
            return full.clone() if self.own_output else full

        return full, finish


def _reduce_dx(dx, group, row_sharded):
    """Start the one collective of the backward.  Returns (work, result): the
    all-reduce works in place; the reduce-scatter leaves this rank's rows of the
    sum in a new (T/P, dm) tensor."""
    if not row_sharded:
        return dist.all_reduce(dx, op=dist.ReduceOp.SUM, group=group, async_op=True), dx
    world = dist.get_world_size(group)
    mine = torch.empty((dx.shape[0] // world, dx.shape[1]), device=dx.device, dtype=dx.dtype)
    return dist.reduce_scatter_tensor(mine, dx, op=dist.ReduceOp.SUM, group=group, async_op=True), mine


class ColumnParallelSwiGLU(Function):
    """``ColumnParallelSwiGLU.apply(x, w_gate_shard, w_up_shard, group=None, fast_accum=False,
    backend=None, row_sharded=False)``.

    Weight shards: (d_model, d_intermediate / world_size).  Returns this rank's
    column slice of out for ALL tokens.

    row_sharded=False: x (bs, sq, d_model) is identical on every rank; the gradient
    returned for x is the full, all-reduced dX.
    row_sharded=True: x (bs/P, sq, d_model) holds this rank's tokens (rank-major in
    the flattened token order); they are all-gathered for the forward and the
    gradient returned for x is this rank's rows of the reduce-scattered dX."""

    @staticmethod
    def forward(ctx, x, w_gate_shard, w_up_shard, group=None, fast_accum=False, backend=None,
                row_sharded=False, reducer=None):
        backend = backend or _CudaBackend
        assert x.ndim == 3 and w_gate_shard.ndim == 2, "Incorrect number of dimensions for LHS or RHS"
        assert w_gate_shard.shape == w_up_shard.shape, "Expected both weight matrices to have same shape"
        assert x.shape[2] == w_up_shard.shape[0], "Dimension mismatch between x and the weight shards"
        bs, sq, dm = x.shape
        x2d = x.contiguous().view(bs * sq, dm)
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        sharded = bool(row_sharded) and world > 1
        if sharded:
            x_all = torch.empty((world * bs * sq, dm), device=x2d.device, dtype=x2d.dtype)
            dist.all_gather_into_tensor(x_all, x2d, group=group)
            x2d = x_all
        wg = w_gate_shard.contiguous()
        wu = w_up_shard.contiguous()
        out, g, u = backend.forward(x2d, wg, wu, fast_accum=fast_accum, save_activations=True)
        ctx.save_for_backward(x2d, wg, wu, g, u)
        ctx.meta = (bs, sq, dm, group, fast_accum, backend, sharded, reducer if world > 1 else None)
        return out.view((world if sharded else 1) * bs, sq, wg.shape[1])

    @staticmethod
    def backward(ctx, grad_output):
        x2d, wg, wu, g, u = ctx.saved_tensors
        bs, sq, dm, group, fast_accum, backend, sharded, reducer = ctx.meta
        dout = grad_output.contiguous().view(x2d.shape[0], wg.shape[1])
        dg, du = backend.gate_grad(dout, g, u)
        if reducer is not None:
            # this library's own reduce-scatter over peer memory: no NCCL kernel needs
            # SMs, so the dW GEMM keeps the whole GPU while the row blocks are gathered
            reducer.scatter(dg, du, wg, wu)
            di_local = wg.shape[1]
            first = reducer.columns_before_reduction(di_local, sharded)
            dwg = dwu = None
            if first > 0:  # GEMM work that absorbs the wait for the slowest peer's dX
                dwg, dwu = backend.grad_weights(x2d, dg, du, fast_accum=fast_accum,
                                                **({} if first == di_local else {"columns": (0, first)}))
            dx, finish = reducer.reduce(sharded)
            if first < di_local:  # ... and the rest of dW beside the gather of the row blocks
                dwg, dwu = backend.grad_weights(x2d, dg, du, fast_accum=fast_accum, out_gate=dwg, out_up=dwu,
                                                columns=(first, di_local - first))
            dx = finish()
            return dx.view(bs, sq, dm), dwg, dwu, None, None, None, None, None
        dx = backend.grad_input(dg, du, wg, wu)
        work = None
        kind = "reduce_scatter" if sharded else "all_reduce"
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            seconds = collective_seconds(dx, group, kind)  # measured on first use, then cached
            work, dx = _reduce_dx(dx, group, sharded)
        if work is not None and hasattr(backend, "grad_weights_beside_collective"):
            dwg, dwu = backend.grad_weights_beside_collective(
                x2d, dg, du, fast_accum=fast_accum, world_size=dist.get_world_size(group), work=work,
                collective=kind, group=group, collective_s=seconds)
        else:
            dwg, dwu = backend.grad_weights(x2d, dg, du, fast_accum=fast_accum)
        if work is not None:
            work.wait()
        return dx.view(bs, sq, dm), dwg, dwu, None, None, None, None, None


def shard_rows(w: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """Contiguous copy of this rank's row slice of a (d_intermediate, d_out) weight -
    the row-parallel partner of shard_columns for the down projection."""
    lo, hi = shard_bounds(w.shape[0], rank, world_size)
    return w[lo:hi].contiguous()


class TensorParallelSwiGLUMLP(Function):
    """``TensorParallelSwiGLUMLP.apply(x, w_gate_shard, w_up_shard, w_down_shard, group=None)``:
    the whole MLP block ``(silu(x@W_gate) * (x@W_up)) @ W_down`` with the usual
    column-parallel / row-parallel pairing.  Rank r holds columns of W_gate, W_up
    and the matching rows of W_down; x is replicated.

    Forward: everything is local up to a partial y, which is all-reduced (one
    collective).  Backward: dW_down, dout, dg/du, dW_gate, dW_up are local; the
    partial dX is all-reduced beside the dW GEMM (one collective).  Returns the full
    y; the gradient for x is the full dX."""

    @staticmethod
    def forward(ctx, x, w_gate_shard, w_up_shard, w_down_shard, group=None, backend=None):
        backend = backend or _CudaBackend
        assert x.ndim == 3 and w_gate_shard.ndim == 2 and w_down_shard.ndim == 2, "Incorrect number of dimensions"
        assert w_gate_shard.shape == w_up_shard.shape, "Expected both weight matrices to have same shape"
        assert x.shape[2] == w_gate_shard.shape[0], "Dimension mismatch between x and the weight shards"
        assert w_gate_shard.shape[1] == w_down_shard.shape[0], "w_down shard must hold the rows matching the column shard"
        bs, sq, dm = x.shape
        x2d = x.contiguous().view(bs * sq, dm)
        wg, wu, wd = w_gate_shard.contiguous(), w_up_shard.contiguous(), w_down_shard.contiguous()
        out, g, u = backend.forward(x2d, wg, wu, fast_accum=False, save_activations=True)
        y = backend.gemm(out, wd)
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
        ctx.save_for_backward(x2d, wg, wu, wd, g, u, out)
        ctx.meta = (bs, sq, dm, group, backend)
        return y.view(bs, sq, wd.shape[1])

    @staticmethod
    def backward(ctx, grad_y):
        x2d, wg, wu, wd, g, u, out = ctx.saved_tensors
        bs, sq, dm, group, backend = ctx.meta
        dy = grad_y.contiguous().view(bs * sq, wd.shape[1])
        dwd = backend.gemm(out, dy, trans_a=True)
        dout = backend.gemm(dy, wd, trans_b=True)
        dg, du = backend.gate_grad(dout, g, u)
        dx = backend.grad_input(dg, du, wg, wu)
        work = None
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            seconds = collective_seconds(dx, group, "all_reduce")
            work = dist.all_reduce(dx, op=dist.ReduceOp.SUM, group=group, async_op=True)
        if work is not None and hasattr(backend, "grad_weights_beside_collective"):
            dwg, dwu = backend.grad_weights_beside_collective(
                x2d, dg, du, fast_accum=False, world_size=dist.get_world_size(group), work=work,
                group=group, collective_s=seconds)
        else:
            dwg, dwu = backend.grad_weights(x2d, dg, du, fast_accum=False)
        if work is not None:
            work.wait()
        return dx.view(bs, sq, dm), dwg, dwu, dwd, None, None


def column_parallel_swiglu(
    x: torch.Tensor, w_gate_shard: torch.Tensor, w_up_shard: torch.Tensor,
    group: Optional[dist.ProcessGroup] = None, fast_accum: bool = False, row_sharded: bool = False,
    backend=None, reducer: Optional["PeerDxReducer"] = None,
) -> torch.Tensor:
    """``reducer``: a PeerDxReducer for this group and (T, d_model): the dX collective is
    then done by this library's kernels over NVLink peer memory instead of NCCL."""
    return ColumnParallelSwiGLU.apply(x, w_gate_shard, w_up_shard, group, fast_accum, backend, row_sharded,
                                      reducer)

"""Sequence-parallel SSD: each rank owns a contiguous slice of the sequence.

The recurrence is a first-order linear scan, so a slice composes as the pair
(total log-decay, final state for a zero entry state).  Forward: every rank runs the local
stages, ONE exchange moves the W small records and folds the records of the ranks before this one
into the state entering its slice (an exclusive prefix scan over ranks), then the rank finishes
locally.  Backward is the mirror image for the state gradient (its exchange runs on a side stream
while the forward recompute pass, which does not need it, runs on the compute stream), plus a sum
of dA / dD over ranks because those parameters are replicated.  The reference has no multi-GPU
path at all (no collective call site anywhere in its tree); this module is new work, not a
counterpart.

On the GPU the exchange is the library's own C entry point (`ssd_sp_exchange_fwd/_bwd`: NCCL
point-to-point transfers into local memory + the prefix kernel), so this file is a thin caller: what a Rust/tch
host does with the same entry points.  `ops` is the set of device operations used; it is a
parameter so that the host-side logic (slice bookkeeping, exchange order, boundary handling, the
rendezvous that detects a missing or disagreeing rank) can be exercised by CPU ranks in tests.

Failure detection (checked mode, `timeout_s` given): before the exchange every rank posts a
signature of its problem to the process group's key-value store and waits, for at most
`timeout_s`, for the others.  A rank that never posts gives SsdError(SSD_ERR_TIMEOUT) on the
ranks that wait for it, ranks that disagree about world size or shapes give
SsdError(SSD_ERR_BAD_SHAPE); in both cases no collective has been entered, so the process group
(and the NCCL communicator) stay usable - the "fail, report, stay usable" shape of the reference's
update loop (trading_bots/src/torch/train/update.rs:190-204).
"""
from __future__ import annotations

import ctypes as C
import datetime
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import _lib as L

SSD_ERR_BAD_SHAPE, SSD_ERR_TIMEOUT = -1, -7

_rendezvous_seq: dict = {}


def rendezvous(signature: tuple, group=None, timeout_s: float = 2.0, tag: Optional[str] = None, store=None) -> None:
    """Host-side check that every rank of `group` is about to enter the same exchange.  Raises
    SsdError(SSD_ERR_TIMEOUT) naming the ranks that did not post within `timeout_s`, SsdError(SSD_ERR_BAD_SHAPE) naming the
    first rank whose signature differs.  Uses only the key-value store: no collective is entered, nothing is left
    half-done.  `tag` names the exchange; without it a per-group call counter is used (ranks must then call in step)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    store = store or dist.distributed_c10d._get_default_store()
    gkey = "world" if group is None else f"g{dist.get_process_group_ranks(group)}"
    if tag is None:
        n = _rendezvous_seq[gkey] = _rendezvous_seq.get(gkey, 0) + 1
        tag = f"n{n}"
    base = f"ssd_sp/{gkey}/{tag}"
    mine = repr(tuple(signature))
    store.set(f"{base}/{rank}", mine)
    keys = [f"{base}/{q}" for q in range(world)]
    try:
        store.wait(keys, datetime.timedelta(seconds=timeout_s))
    except Exception as e:   # DistStoreError / RuntimeError, by torch version
        missing = [q for q in range(world) if not store.check([keys[q]])]
        if not missing:      # they arrived between the timeout and the check
            missing = []
        else:
            raise L.SsdError(SSD_ERR_TIMEOUT, f"sequence-parallel exchange {tag!r}: rank(s) {missing} of {world} did not post within "
                                              f"{timeout_s} s; no collective was entered ({type(e).__name__})") from None
    for q in range(world):
        theirs = store.get(keys[q]).decode()
        if theirs != mine:
            raise L.SsdError(SSD_ERR_BAD_SHAPE, f"sequence-parallel exchange {tag!r}: rank {q} posted {theirs}, rank {rank} has {mine} "
                                                "(world size, shapes, dtype and direction must agree); no collective was entered")


def _gather(states: torch.Tensor, logdecay: torch.Tensor, group, world: int):
    """One torch.distributed collective for both records: pack [state | logdecay] per (batch, head)."""
    Bn, H, P, N = states.shape
    packed = torch.cat([states.reshape(Bn * H, P * N), logdecay.reshape(Bn * H, 1)], dim=1).contiguous()
    flat = torch.empty(world * packed.shape[0], packed.shape[1], dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(flat, packed, group=group)
    out = flat.view(world, Bn * H, P * N + 1)
    gs = out[:, :, : P * N].reshape(world, Bn, H, P, N).contiguous()
    gl = out[:, :, P * N].reshape(world, Bn, H).contiguous()
    return gs, gl


class SpOps:
    """Operations `sp_forward` / `sp_backward` are written against.  This base class does the exchange with
    torch.distributed collectives on whatever backend the group has (gloo ranks in the CPU tests); subclasses provide
    forward / backward / total_logdecay / prefix_state."""

    def exchange(self, direction, local_total, boundary, tensors, chunk, algo, workspace, group, overlap: Optional[Callable] = None):
        x, dt, A, Bm, Cm, D, z = tensors
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        logdecay = self.total_logdecay(x, dt, A, Bm, Cm, z, chunk, algo, workspace)
        gs, gl = _gather(local_total, logdecay, group, world)
        if overlap is not None:
            overlap()
        return self.prefix_state(gs, gl, world, rank, direction, boundary)

    def allreduce_params(self, dA, dD, group):
        packed = torch.cat([dA, dD]) if dD is not None else dA.clone()
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
        H = dA.numel()
        return packed[:H].clone(), (packed[H:].clone() if dD is not None else None)


class CudaOps(SpOps):
    """Device operations backed by the C ABI, the exchange included (NCCL inside the library)."""

    def __init__(self):
        self._comms = {}
        self._side = {}

    def forward(self, stages, x, dt, A, Bm, Cm, D, z, init_state, chunk, algo, workspace, y, final_state):
        from .ssd import forward
        return forward(x, dt, A, Bm, Cm, D, z, init_state, chunk=chunk, algo=algo, workspace=workspace, y=y,
                       final_state=final_state, for_backward=True, stages=stages)

    def backward(self, stages, dy, x, dt, A, Bm, Cm, D, z, init_state, dfinal, chunk, algo, workspace, out):
        from .ssd import backward
        return backward(dy, x, dt, A, Bm, Cm, D, z, init_state, dfinal, chunk=chunk, algo=algo,
                        workspace=workspace, fwd_saved=True, want_dinit=True, stages=stages, out=out)

    def total_logdecay(self, x, dt, A, Bm, Cm, z, chunk, algo, workspace):
        from .ssd import _ptr, _stream, make_dims
        d = make_dims(x, dt, Bm, Cm, chunk, z=z, algo=algo)
        out = torch.empty(d.batch, d.nheads, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            L.check(L.load().ssd_sp_total_logdecay(C.byref(d), _ptr(workspace), workspace.numel(), _ptr(out),
                                                   _stream(x.device)))
        return out

    def prefix_state(self, gathered_states, gathered_logdecay, world, rank, direction, boundary):
        from .ssd import _ptr, _stream
        W, Bn, H, P, N = gathered_states.shape
        out = torch.empty(Bn, H, P, N, dtype=torch.float32, device=gathered_states.device)
        dev = gathered_states.device
        with torch.cuda.device(dev):
            L.check(L.load().ssd_sp_prefix_state(_ptr(gathered_states), _ptr(gathered_logdecay), world, rank,
                                                 direction, Bn * H, P * N, _ptr(boundary), _ptr(out), _stream(dev)))
        return out

    # ---- the library's own exchange ------------------------------------------------------------------------------
    def comm(self, group, device):
        """The library's communicator for `group` on `device` (made once: rank 0 draws the NCCL id, torch.distributed
        carries it to the others - the one thing the host program has to move by its own means)."""
        key = (None if group is None else tuple(dist.get_process_group_ranks(group)), device.index)
        if key in self._comms:
            return self._comms[key]
        lib = L.load()
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        ident = (C.c_ubyte * L.SP_UNIQUE_ID_BYTES)()
        if rank == 0:
            L.check(lib.ssd_sp_unique_id(ident))
        box = [bytes(ident)]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        ident = (C.c_ubyte * L.SP_UNIQUE_ID_BYTES).from_buffer_copy(box[0])
        with torch.cuda.device(device):
            h = lib.ssd_sp_comm_new(ident, world, rank)
        if not h:
            raise L.SsdError(-5, lib.ssd_last_error().decode())
        self._comms[key] = h
        return h

    def close(self):
        for h in self._comms.values():
            L.load().ssd_sp_comm_free(h)
        self._comms.clear()

    def exchange(self, direction, local_total, boundary, tensors, chunk, algo, workspace, group, overlap=None, timeout_ms=0):
        from .ssd import _ptr, make_dims
        x, dt, A, Bm, Cm, D, z = tensors
        dev = x.device
        lib = L.load()
        d = make_dims(x, dt, Bm, Cm, chunk, z=z, algo=algo)
        world = dist.get_world_size(group)
        h = self.comm(group, dev)
        nbytes = lib.ssd_sp_exchange_bytes(C.byref(d), world)
        exch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        out = torch.empty_like(local_total)
        fn = lib.ssd_sp_exchange_fwd if direction > 0 else lib.ssd_sp_exchange_bwd
        cur = torch.cuda.current_stream(dev)
        if overlap is None:
            with torch.cuda.device(dev):
                L.check(fn(C.byref(d), _ptr(workspace), workspace.numel(), h, _ptr(local_total), _ptr(boundary), _ptr(out),
                           _ptr(exch), nbytes, C.c_void_p(cur.cuda_stream), timeout_ms))
            return out
        # the exchange on a side stream, `overlap` (local work that does not need its result) on the compute stream
        side = self._side.setdefault(dev.index, torch.cuda.Stream(dev))
        side.wait_stream(cur)
        with torch.cuda.device(dev):
            L.check(fn(C.byref(d), _ptr(workspace), workspace.numel(), h, _ptr(local_total), _ptr(boundary), _ptr(out),
                       _ptr(exch), nbytes, C.c_void_p(side.cuda_stream), timeout_ms))
        for t in (exch, out, local_total):
            t.record_stream(side)
        overlap()
        cur.wait_stream(side)
        return out

    def allreduce_params(self, dA, dD, group, timeout_ms=0):
        from .ssd import _ptr, _stream
        dev = dA.device
        h = self.comm(group, dev)
        with torch.cuda.device(dev):
            L.check(L.load().ssd_sp_allreduce_params(h, _ptr(dA), _ptr(dD), dA.numel(), _stream(dev), timeout_ms))
        return dA, dD


_default_ops: Optional[CudaOps] = None


def default_ops() -> CudaOps:
    """One CudaOps per process, so that the library's communicators are made once."""
    global _default_ops
    if _default_ops is None:
        _default_ops = CudaOps()
    return _default_ops


def slice_bounds(seqlen: int, world: int, rank: int, chunk: int):
    """Contiguous [start, end) of `rank`; every slice but the last is a whole number of chunks."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad world/rank {world}/{rank}")
    nchunks = (seqlen + chunk - 1) // chunk
    per = (nchunks + world - 1) // world
    start = min(seqlen, rank * per * chunk)
    end = min(seqlen, (rank + 1) * per * chunk)
    if end <= start:
        raise ValueError(f"rank {rank} of {world} gets an empty slice of seqlen {seqlen} at chunk {chunk}")
    return start, end


@dataclass
class SpContext:
    tensors: tuple
    workspace: torch.Tensor
    state_in: Optional[torch.Tensor]
    chunk: int
    algo: str
    world: int
    rank: int
    group: object = None
    timeout_s: Optional[float] = None
    extra: dict = field(default_factory=dict)


def _signature(direction, world, x, Bm, chunk):
    return ("ssd_sp", direction, world, x.shape[0], x.shape[2], x.shape[3], Bm.shape[2], Bm.shape[3], chunk, str(x.dtype))


def sp_forward(x, dt, A, Bm, Cm, D=None, z=None, init_state=None, *, chunk, algo="auto", group=None, ops=None,
               timeout_s: Optional[float] = None, tag: Optional[str] = None):
    """Forward on this rank's slice.  `init_state` is the state entering the GLOBAL sequence (same
    tensor on every rank, or None).  Returns (y_local, state_at_slice_end, ctx).  `timeout_s` switches the checked
    mode on (see the module text)."""
    ops = ops or default_ops()
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if timeout_s is not None:
        rendezvous(_signature(+1, world, x, Bm, chunk), group, timeout_s, None if tag is None else tag + "/fwd")
    tensors = (x, dt, A, Bm, Cm, D, z)
    y, total, ws = ops.forward(L.STAGE_LOCAL | L.STAGE_TOTAL, x, dt, A, Bm, Cm, D, z, None, chunk, algo, None, None, None)
    kw = {"timeout_ms": int(timeout_s * 1000)} if (timeout_s is not None and isinstance(ops, CudaOps)) else {}
    state_in = ops.exchange(+1, total, init_state, tensors, chunk, algo, ws, group, **kw)
    y, fin, ws = ops.forward(L.STAGE_FINISH, x, dt, A, Bm, Cm, D, z, state_in, chunk, algo, ws, y, total)
    ctx = SpContext(tensors, ws, state_in, chunk, algo, world, rank, group, timeout_s, {"tag": tag})
    return y, fin, ctx


def sp_backward(dy, ctx: SpContext, dfinal_state=None, *, ops=None):
    """Backward on this rank's slice.  `dfinal_state` is the gradient w.r.t. the GLOBAL final state
    (same tensor on every rank, or None).  dA and dD come back summed over ranks."""
    ops = ops or default_ops()
    x, dt, A, Bm, Cm, D, z = ctx.tensors
    if ctx.timeout_s is not None:
        tag = ctx.extra.get("tag")
        rendezvous(_signature(-1, ctx.world, x, Bm, ctx.chunk), ctx.group, ctx.timeout_s, None if tag is None else tag + "/bwd")
    out = {}
    args = (dy, x, dt, A, Bm, Cm, D, z, ctx.state_in)
    g = ops.backward(L.STAGE_LOCAL_STATES | L.STAGE_TOTAL, *args, None, ctx.chunk, ctx.algo, ctx.workspace, out)
    rest = lambda: ops.backward(L.STAGE_LOCAL_REST, *args, None, ctx.chunk, ctx.algo, ctx.workspace, out)
    kw = {"timeout_ms": int(ctx.timeout_s * 1000)} if (ctx.timeout_s is not None and isinstance(ops, CudaOps)) else {}
    dstate_out = ops.exchange(-1, g["dinit"], dfinal_state, ctx.tensors, ctx.chunk, ctx.algo, ctx.workspace, ctx.group,
                              overlap=rest, **kw)
    g = ops.backward(L.STAGE_FINISH, *args, dstate_out, ctx.chunk, ctx.algo, ctx.workspace, out)
    g["dA"], dD = ops.allreduce_params(g["dA"], g.get("dD") if D is not None else None, ctx.group)
    if D is not None:
        g["dD"] = dD
    return g

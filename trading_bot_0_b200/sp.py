"""Sequence-parallel SSD: each rank owns a contiguous slice of the sequence.

The recurrence is a first-order linear scan, so a slice composes as the pair
(total log-decay, final state for a zero entry state).  Forward: every rank runs the local
stages, one all-gather moves the W small records, each rank folds the records of the ranks
before it into the state entering its slice (an exclusive prefix scan over ranks), then finishes
locally.  Backward is the mirror image for the state gradient, plus a sum of dA / dD over ranks
because those parameters are replicated.  The reference has no multi-GPU path at all (no
collective call site anywhere in its tree); this module is new work, not a counterpart.

`ops` is the set of device operations used; the default binds the CUDA library.  It is a
parameter so the host-side logic (slice bookkeeping, gather order, boundary handling) can be
exercised by CPU ranks in tests.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib as L


class CudaOps:
    """Device operations backed by the C ABI."""

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


def _gather(states: torch.Tensor, logdecay: torch.Tensor, group, world: int):
    """One collective for both records: pack [state | logdecay] per (batch, head)."""
    Bn, H, P, N = states.shape
    packed = torch.cat([states.reshape(Bn * H, P * N), logdecay.reshape(Bn * H, 1)], dim=1).contiguous()
    flat = torch.empty(world * packed.shape[0], packed.shape[1], dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(flat, packed, group=group)
    out = flat.view(world, Bn * H, P * N + 1)
    gs = out[:, :, : P * N].reshape(world, Bn, H, P, N).contiguous()
    gl = out[:, :, P * N].reshape(world, Bn, H).contiguous()
    return gs, gl


@dataclass
class SpContext:
    tensors: tuple
    workspace: torch.Tensor
    state_in: Optional[torch.Tensor]
    gathered_logdecay: torch.Tensor
    chunk: int
    algo: str
    world: int
    rank: int
    group: object = None
    extra: dict = field(default_factory=dict)


def sp_forward(x, dt, A, Bm, Cm, D=None, z=None, init_state=None, *, chunk, algo="auto", group=None, ops=None):
    """Forward on this rank's slice.  `init_state` is the state entering the GLOBAL sequence (same
    tensor on every rank, or None).  Returns (y_local, state_at_slice_end, ctx)."""
    ops = ops or CudaOps()
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    y, total, ws = ops.forward(L.STAGE_LOCAL | L.STAGE_TOTAL, x, dt, A, Bm, Cm, D, z, None, chunk, algo, None, None, None)
    logdecay = ops.total_logdecay(x, dt, A, Bm, Cm, z, chunk, algo, ws)
    gs, gl = _gather(total, logdecay, group, world)
    state_in = ops.prefix_state(gs, gl, world, rank, +1, init_state)
    y, fin, ws = ops.forward(L.STAGE_FINISH, x, dt, A, Bm, Cm, D, z, state_in, chunk, algo, ws, y, total)
    ctx = SpContext((x, dt, A, Bm, Cm, D, z), ws, state_in, gl, chunk, algo, world, rank, group)
    return y, fin, ctx


def sp_backward(dy, ctx: SpContext, dfinal_state=None, *, ops=None):
    """Backward on this rank's slice.  `dfinal_state` is the gradient w.r.t. the GLOBAL final state
    (same tensor on every rank, or None).  dA and dD come back summed over ranks."""
    ops = ops or CudaOps()
    x, dt, A, Bm, Cm, D, z = ctx.tensors
    out = {}
    g = ops.backward(L.STAGE_LOCAL | L.STAGE_TOTAL, dy, x, dt, A, Bm, Cm, D, z, ctx.state_in, None, ctx.chunk,
                     ctx.algo, ctx.workspace, out)
    gs, _ = _gather(g["dinit"], ctx.gathered_logdecay[ctx.rank], ctx.group, ctx.world)
    dstate_out = ops.prefix_state(gs, ctx.gathered_logdecay, ctx.world, ctx.rank, -1, dfinal_state)
    g = ops.backward(L.STAGE_FINISH, dy, x, dt, A, Bm, Cm, D, z, ctx.state_in, dstate_out, ctx.chunk, ctx.algo,
                     ctx.workspace, out)
    packed = torch.cat([g["dA"], g["dD"]]) if D is not None else g["dA"].clone()
    dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=ctx.group)
    H = g["dA"].numel()
    g["dA"] = packed[:H].clone()
    if D is not None:
        g["dD"] = packed[H:].clone()
    return g

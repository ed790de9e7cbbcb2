"""Recurrent-state container for streamed rollout.

Shaped after the reference's stream API: `StreamState` (trading_bots/src/torch/model/trading_model.rs:56-75),
`init_stream_state_batched` (trading_bots/src/torch/model/stream/state.rs:103-105), `reset`
(stream/state.rs:10-20), the env-indexed reset that avoids a host sync
(trading_bots/src/torch/model/stream/live.rs:114-158) and `detach_stream_state`
(stream/state.rs:24-30).  The state is an ordinary caller-owned fp32 tensor; the step kernel
updates it in place.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from .ssd import _ptr, _stream, state_update


class StreamState:
    def __init__(self, state: torch.Tensor):
        if state.dim() != 4 or state.dtype != torch.float32 or not state.is_contiguous():
            raise ValueError("state must be a contiguous float32 [streams, nheads, headdim, dstate] tensor")
        self.state = state

    @property
    def streams(self) -> int:
        return self.state.shape[0]

    def reset(self) -> None:
        """Zero every stream (start of a rollout)."""
        self.state.zero_()

    def reset_streams(self, stream_idx: torch.Tensor) -> None:
        """Zero the rows listed in `stream_idx` (device int64 tensor) with one kernel and no host
        sync: the count comes from the tensor's shape, never from its contents."""
        if stream_idx.numel() == 0:
            return
        if not stream_idx.is_cuda:
            raise ValueError("stream_idx must be a CUDA tensor (there is no CPU path)")
        idx = stream_idx.to(device=self.state.device, dtype=torch.int64).contiguous()
        row = self.state[0].numel()
        dev = self.state.device
        with torch.cuda.device(dev):
            L.check(L.load().ssd_state_reset_rows(_ptr(self.state), row, _ptr(idx), idx.numel(),
                                                  self.streams, _stream(dev)))

    def detach(self) -> "StreamState":
        """Cut the state loose from any graph between rollouts."""
        self.state = self.state.detach()
        return self

    def step(self, x, dt, A, Bm, Cm, D=None, z=None, *, y=None):
        """Advance every stream by one timestep; returns y [streams, nheads, headdim]."""
        return state_update(self.state, x, dt, A, Bm, Cm, D, z, y=y)


def init_stream_state_batched(streams: int, nheads: int, headdim: int, dstate: int, device, *, std: float = 0.0,
                              generator=None) -> StreamState:
    """Zero state, or N(0, std) when std > 0 (the rollout workload draws N(0, 0.1))."""
    st = torch.zeros(streams, nheads, headdim, dstate, dtype=torch.float32, device=device)
    if std > 0:
        st.normal_(0.0, std, generator=generator)
    return StreamState(st)

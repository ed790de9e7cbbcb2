"""B200-native Mamba-2 SSD operator behind the trading_bot_0 operator surface."""
from . import _lib
from .ssd import (alloc_workspace, backward, forward, make_dims, ssd_scan, state_update, workspace_bytes)
from .stream import StreamState, init_stream_state_batched
from . import sp

__all__ = ["forward", "backward", "state_update", "ssd_scan", "make_dims", "workspace_bytes",
           "alloc_workspace", "StreamState", "init_stream_state_batched", "_lib"]

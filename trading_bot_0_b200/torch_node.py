"""The libtorch (C++) autograd node of the SSD operator, driven from Python.

`libssd_b200_torch.so` holds a `torch::autograd::Function` over the C ABI plus C entry points in the calling convention
of the libtch shim that tch-rs binds (csrc/ssd_torch.cpp).  It also registers `torch.ops.ssd_b200.scan` /
`torch.ops.ssd_b200.state_update`, which is how this module and the tests reach the same node a Rust caller would.
"""
from __future__ import annotations

import torch

from .build import TORCH_LIB
from .ssd import ALGOS

_loaded = False


def load() -> None:
    global _loaded
    if _loaded:
        return
    if not TORCH_LIB.exists():
        raise ImportError(f"{TORCH_LIB} is missing: run `python -m trading_bot_0_b200.build --torch`. There is no fallback.")
    torch.ops.load_library(str(TORCH_LIB))
    _loaded = True


def ssd_scan(x, dt, A, Bm, Cm, D=None, z=None, init_state=None, *, chunk=128, algo="auto", dt_bias=None, dt_softplus=False):
    """Differentiable SSD through the C++ node: returns (y, final_state)."""
    load()
    return torch.ops.ssd_b200.scan(x, dt, A, Bm, Cm, D, z, init_state, dt_bias, chunk, dt_softplus, ALGOS[algo])


def state_update(state, x, dt, A, Bm, Cm, D=None, z=None, *, dt_bias=None, dt_softplus=False):
    """One timestep over all streams, in place on `state`; returns y."""
    load()
    return torch.ops.ssd_b200.state_update(state, x, dt, A, Bm, Cm, D, z, dt_bias, dt_softplus)

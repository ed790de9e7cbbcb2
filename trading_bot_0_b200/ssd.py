"""Tensor-in / tensor-out host side of the SSD operator.

Mirrors the safe wrapper a tch caller would write over the C ABI: validate first and raise
(`validate` in trading_bots/src/torch/fa4.rs:145-191 checks rank, device, dtype, unit inner
stride and matching batch before its FFI call), then pass raw device pointers, a caller-owned
workspace and the current stream.  Explicit `forward` / `backward` calls are the contract
(tch-rs has no custom autograd node); `ssd_scan` additionally wraps them in a
torch.autograd.Function so they take part in `loss.backward()`.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib as L

_DT = {torch.float32: L.SSD_F32, torch.bfloat16: L.SSD_BF16}
ALGOS = {"auto": L.ALGO_AUTO, "fp32_cores": L.ALGO_FP32_CORES, "tensor": L.ALGO_TENSOR,
         "tensor_onetile": L.ALGO_TENSOR_ONETILE}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _need(cond: bool, msg: str):
    if not cond:
        raise ValueError(msg)


def _check_seq(name, t, shape, dtype, device):
    _need(t.dim() == len(shape), f"{name}: expected rank {len(shape)}, got {t.dim()}")
    _need(tuple(t.shape) == tuple(shape), f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")
    _need(t.dtype == dtype, f"{name}: expected dtype {dtype}, got {t.dtype}")
    _need(t.device == device, f"{name}: expected device {device}, got {t.device}")
    _need(t.stride(-1) == 1, f"{name}: innermost stride must be 1")
    if t.dim() == 4:
        _need(t.stride(2) == t.shape[3], f"{name}: the last two dims must be dense")


def _check_dense_f32(name, t, shape, device):
    _need(tuple(t.shape) == tuple(shape), f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")
    _need(t.dtype == torch.float32, f"{name}: expected float32, got {t.dtype}")
    _need(t.device == device and t.is_contiguous(), f"{name}: must be a contiguous tensor on {device}")


def make_dims(x, dt, Bm, Cm, chunk, *, z=None, y=None, algo="auto", dt_softplus=False) -> L.SsdDims:
    """Validate the sequence operands and fill the geometry struct."""
    _need(x.is_cuda, "x must be a CUDA tensor (there is no CPU path)")
    _need(x.dim() == 4, "x must be [batch, seqlen, nheads, headdim]")
    _need(x.dtype in _DT, f"unsupported dtype {x.dtype}")
    Bn, Ln, H, P = x.shape
    _need(Bm.dim() == 4, "B must be [batch, seqlen, ngroups, dstate]")
    G, N = Bm.shape[2], Bm.shape[3]
    dev = x.device
    _check_seq("x", x, (Bn, Ln, H, P), x.dtype, dev)
    _check_seq("dt", dt, (Bn, Ln, H), x.dtype, dev)
    _check_seq("B", Bm, (Bn, Ln, G, N), x.dtype, dev)
    _check_seq("C", Cm, (Bn, Ln, G, N), x.dtype, dev)
    _need(H % G == 0, f"nheads ({H}) must be a multiple of ngroups ({G})")
    _need(1 <= chunk <= 256, f"chunk must be in [1, 256], got {chunk}")
    d = L.SsdDims()
    d.batch, d.seqlen, d.nheads, d.headdim, d.dstate, d.ngroups, d.chunk = Bn, Ln, H, P, N, G, chunk
    d.dtype, d.algo, d.device = _DT[x.dtype], ALGOS[algo], dev.index if dev.index is not None else torch.cuda.current_device()
    d.has_z = 0 if z is None else 1
    d.dt_softplus = 1 if dt_softplus else 0
    d.x_stride_b, d.x_stride_l = x.stride(0), x.stride(1)
    d.dt_stride_b, d.dt_stride_l = dt.stride(0), dt.stride(1)
    d.b_stride_b, d.b_stride_l = Bm.stride(0), Bm.stride(1)
    d.c_stride_b, d.c_stride_l = Cm.stride(0), Cm.stride(1)
    if z is not None:
        _check_seq("z", z, (Bn, Ln, H, P), x.dtype, dev)
        d.z_stride_b, d.z_stride_l = z.stride(0), z.stride(1)
    if y is not None:
        _check_seq("y/dy", y, (Bn, Ln, H, P), x.dtype, dev)
        d.y_stride_b, d.y_stride_l = y.stride(0), y.stride(1)
    return d


def workspace_bytes(dims: L.SsdDims, backward: bool = False) -> int:
    n = L.load().ssd_workspace_bytes(C.byref(dims), L.PASS_BWD if backward else L.PASS_FWD)
    if n == 0:
        raise L.SsdError(-1, L.load().ssd_last_error().decode())
    return n


def alloc_workspace(dims: L.SsdDims, device, backward: bool = False) -> torch.Tensor:
    return torch.empty(workspace_bytes(dims, backward), dtype=torch.uint8, device=device)


def workspace_status(workspace: torch.Tensor) -> int:
    """Wait for the current stream and read the status word of `workspace`: 0 when healthy; raises SsdError (code
    SSD_ERR_TIMEOUT, wait-site in the message) when a bounded wait inside a pipelined kernel ran out.  The device-side
    counterpart of the error read the reference makes after every FFI call (trading_bots/src/torch/cuda/graph.rs:107-118)."""
    code = C.c_int32(0)
    with torch.cuda.device(workspace.device):
        L.check(L.load().ssd_workspace_status(_ptr(workspace), _stream(workspace.device), C.byref(code)))
    return int(code.value)


def _out_slot(o, key, shape, dtype, dev):
    """A caller-provided output must be dense, 16-byte aligned and of the right shape; a missing one is allocated."""
    t = o.get(key)
    if t is None:
        o[key] = torch.empty(*shape, dtype=dtype, device=dev)
        return
    _need(tuple(t.shape) == tuple(shape) and t.dtype == dtype and t.device == dev,
          f"out[{key!r}]: expected {tuple(shape)} {dtype} on {dev}, got {tuple(t.shape)} {t.dtype} on {t.device}")
    _need(t.is_contiguous() and t.data_ptr() % 16 == 0, f"out[{key!r}]: must be contiguous and 16-byte aligned")


def forward(x, dt, A, Bm, Cm, D=None, z=None, init_state=None, *, chunk, algo="auto", workspace=None,
            y=None, final_state=None, return_final_state=True, for_backward=False, stages=None,
            dt_bias=None, dt_softplus=False, check=False):
    """y, final_state, workspace = SSD(x, dt, A, B, C, D, z, init_state).  With `dt_bias` / `dt_softplus` the step
    size is act(dt + dt_bias), evaluated inside the cumsum kernel (the pre-activation of a Mamba-2 layer).
    `check=True` waits for the stream afterwards and raises if a kernel reported a timed-out wait."""
    lib = L.load()
    dev = x.device
    if y is None:
        y = torch.empty_like(x, memory_format=torch.contiguous_format)
    d = make_dims(x, dt, Bm, Cm, chunk, z=z, y=y, algo=algo, dt_softplus=dt_softplus)
    H, P, N = d.nheads, d.headdim, d.dstate
    _check_dense_f32("A", A, (H,), dev)
    if D is not None:
        _check_dense_f32("D", D, (H,), dev)
    if dt_bias is not None:
        _check_dense_f32("dt_bias", dt_bias, (H,), dev)
    if init_state is not None:
        _check_dense_f32("init_state", init_state, (d.batch, H, P, N), dev)
    if final_state is None and return_final_state:
        final_state = torch.empty(d.batch, H, P, N, dtype=torch.float32, device=dev)
    if final_state is not None:
        _check_dense_f32("final_state", final_state, (d.batch, H, P, N), dev)
    if workspace is None:
        workspace = alloc_workspace(d, dev, backward=for_backward)
    p = L.SsdFwdPtrs(_ptr(x), _ptr(dt), _ptr(A), _ptr(Bm), _ptr(Cm), _ptr(D), _ptr(z), _ptr(init_state),
                     _ptr(y), _ptr(final_state), _ptr(dt_bias))
    with torch.cuda.device(dev):
        if stages is None:
            rc = lib.ssd_forward(C.byref(d), C.byref(p), _ptr(workspace), workspace.numel(), _stream(dev))
        else:
            rc = lib.ssd_forward_staged(C.byref(d), C.byref(p), _ptr(workspace), workspace.numel(), _stream(dev), stages)
    L.check(rc)
    if check:
        workspace_status(workspace)
    return y, final_state, workspace


def backward(dy, x, dt, A, Bm, Cm, D=None, z=None, init_state=None, dfinal_state=None, *, chunk, algo="auto",
             workspace=None, fwd_saved=False, want_dinit=False, stages=None, out=None, dt_bias=None,
             dt_softplus=False, check=False):
    """Gradients of `forward`.  Returns a dict with dx, ddt, dA, dB, dC, dD, dz, dinit (and ddt_bias when dt_bias is
    given; ddt is then the gradient w.r.t. the dt passed in, before bias and activation)."""
    lib = L.load()
    dev = x.device
    d = make_dims(x, dt, Bm, Cm, chunk, z=z, y=dy, algo=algo, dt_softplus=dt_softplus)
    Bn, Ln, H, P, N, G = d.batch, d.seqlen, d.nheads, d.headdim, d.dstate, d.ngroups
    _check_dense_f32("A", A, (H,), dev)
    if D is not None:
        _check_dense_f32("D", D, (H,), dev)
    if init_state is not None:
        _check_dense_f32("init_state", init_state, (Bn, H, P, N), dev)
    if dfinal_state is not None:
        _check_dense_f32("dfinal_state", dfinal_state, (Bn, H, P, N), dev)
    o = out if out is not None else {}
    _out_slot(o, "dx", (Bn, Ln, H, P), x.dtype, dev)
    _out_slot(o, "ddt", (Bn, Ln, H), torch.float32, dev)
    _out_slot(o, "dA", (H,), torch.float32, dev)
    _out_slot(o, "dB", (Bn, Ln, G, N), x.dtype, dev)
    _out_slot(o, "dC", (Bn, Ln, G, N), x.dtype, dev)
    if D is not None:
        _out_slot(o, "dD", (H,), torch.float32, dev)
    if z is not None:
        _out_slot(o, "dz", (Bn, Ln, H, P), x.dtype, dev)
    if want_dinit or init_state is not None:
        _out_slot(o, "dinit", (Bn, H, P, N), torch.float32, dev)
    if dt_bias is not None:
        _check_dense_f32("dt_bias", dt_bias, (H,), dev)
        _out_slot(o, "ddt_bias", (H,), torch.float32, dev)
    if workspace is None:
        _need(not fwd_saved, "fwd_saved=True needs the workspace the forward ran in")
        workspace = alloc_workspace(d, dev, backward=True)
    p = L.SsdBwdPtrs(_ptr(x), _ptr(dt), _ptr(A), _ptr(Bm), _ptr(Cm), _ptr(D), _ptr(z), _ptr(init_state),
                     _ptr(dy), _ptr(dfinal_state), _ptr(o["dx"]), _ptr(o["ddt"]), _ptr(o["dA"]), _ptr(o["dB"]),
                     _ptr(o["dC"]), _ptr(o.get("dD")), _ptr(o.get("dz")), _ptr(o.get("dinit")),
                     1 if fwd_saved else 0, _ptr(dt_bias), _ptr(o.get("ddt_bias")))
    with torch.cuda.device(dev):
        if stages is None:
            rc = lib.ssd_backward(C.byref(d), C.byref(p), _ptr(workspace), workspace.numel(), _stream(dev))
        else:
            rc = lib.ssd_backward_staged(C.byref(d), C.byref(p), _ptr(workspace), workspace.numel(), _stream(dev), stages)
    L.check(rc)
    if check:
        workspace_status(workspace)
    o["workspace"] = workspace
    return o


def state_update(state, x, dt, A, Bm, Cm, D=None, z=None, *, y=None, dt_bias=None, dt_softplus=False):
    """One timestep over all streams, IN PLACE on `state` [S,H,P,N] fp32.  Returns y [S,H,P].  The step size is
    act(dt + dt_bias) as in `forward`."""
    lib = L.load()
    _need(state.is_cuda, "state must be a CUDA tensor (there is no CPU path)")
    dev = state.device
    _need(state.dim() == 4 and state.dtype == torch.float32 and state.is_contiguous(),
          "state must be a contiguous float32 [streams, nheads, headdim, dstate] tensor")
    S, H, P, N = state.shape
    _need(x.dtype in _DT, f"unsupported dtype {x.dtype}")
    _need(Bm.dim() == 3 and Bm.shape[0] == S and Bm.shape[2] == N, "B must be [streams, ngroups, dstate]")
    G = Bm.shape[1]
    _need(H % G == 0, f"nheads ({H}) must be a multiple of ngroups ({G})")
    for name, t, shape in (("x", x, (S, H, P)), ("dt", dt, (S, H)), ("B", Bm, (S, G, N)), ("C", Cm, (S, G, N))):
        _need(tuple(t.shape) == shape and t.dtype == x.dtype and t.device == dev, f"{name}: expected {shape} {x.dtype} on {dev}")
        _need(t.stride(-1) == 1 and (t.dim() < 3 or t.stride(1) == t.shape[2]), f"{name}: inner dims must be dense")
    _check_dense_f32("A", A, (H,), dev)
    if D is not None:
        _check_dense_f32("D", D, (H,), dev)
    if y is None:
        y = torch.empty(S, H, P, dtype=x.dtype, device=dev)
    d = L.SsdStepDims()
    d.streams, d.nheads, d.headdim, d.dstate, d.ngroups = S, H, P, N, G
    d.dtype, d.device = _DT[x.dtype], dev.index if dev.index is not None else torch.cuda.current_device()
    d.dt_softplus = 1 if dt_softplus else 0
    if dt_bias is not None:
        _check_dense_f32("dt_bias", dt_bias, (H,), dev)
    d.x_stride_s, d.dt_stride_s, d.b_stride_s, d.c_stride_s, d.y_stride_s = (
        x.stride(0), dt.stride(0), Bm.stride(0), Cm.stride(0), y.stride(0))
    if z is not None:
        _need(tuple(z.shape) == (S, H, P) and z.dtype == x.dtype and z.device == dev, "z: expected x's shape/dtype/device")
        d.z_stride_s = z.stride(0)
    p = L.SsdStepPtrs(_ptr(state), _ptr(x), _ptr(dt), _ptr(A), _ptr(Bm), _ptr(Cm), _ptr(D), _ptr(z), _ptr(y),
                      _ptr(dt_bias))
    with torch.cuda.device(dev):
        L.check(lib.ssd_state_update(C.byref(d), C.byref(p), _stream(dev)))
    return y


class _SsdScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt, A, Bm, Cm, D, z, init_state, chunk, algo, dt_bias, dt_softplus):
        y, fin, ws = forward(x, dt, A, Bm, Cm, D, z, init_state, chunk=chunk, algo=algo, for_backward=True,
                             dt_bias=dt_bias, dt_softplus=dt_softplus)
        ctx.save_for_backward(x, dt, A, Bm, Cm, D, z, init_state, ws, dt_bias)
        ctx.chunk, ctx.algo, ctx.dt_softplus = chunk, algo, dt_softplus
        return y, fin

    @staticmethod
    def backward(ctx, dy, dfin):
        x, dt, A, Bm, Cm, D, z, init_state, ws, dt_bias = ctx.saved_tensors
        if dy.stride(-1) != 1 or dy.stride(2) != dy.shape[3]:
            dy = dy.contiguous()
        g = backward(dy, x, dt, A, Bm, Cm, D, z, init_state,
                     None if dfin is None else dfin.contiguous(), chunk=ctx.chunk, algo=ctx.algo,
                     workspace=ws, fwd_saved=True, want_dinit=init_state is not None, dt_bias=dt_bias,
                     dt_softplus=ctx.dt_softplus)
        return (g["dx"], g["ddt"].to(dt.dtype), g["dA"], g["dB"], g["dC"], g.get("dD"), g.get("dz"),
                g.get("dinit"), None, None, g.get("ddt_bias"), None)


def ssd_scan(x, dt, A, Bm, Cm, D=None, z=None, init_state=None, *, chunk=128, algo="auto", dt_bias=None,
             dt_softplus=False):
    """Differentiable SSD: returns (y, final_state)."""
    return _SsdScan.apply(x, dt, A, Bm, Cm, D, z, init_state, chunk, algo, dt_bias, dt_softplus)

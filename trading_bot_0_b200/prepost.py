"""The operators either side of the scan in a Mamba-2 layer: causal depthwise conv1d (+ silu) over the
(x | B | C) channels before it, RMS norm of the gated output after it, each with its backward, plus a
differentiable composition of the whole mixer core (`mamba2_mixer_core`).

The step-size activation softplus(dt + dt_bias) and the gate y * silu(z) are not here: they run inside
the scan's own kernels (`ssd.forward(..., dt_bias=, dt_softplus=)`, `z=`).  Reference anchors: the 3-tap
causal depthwise convolution on q/k/v (trading_bots/src/torch/model/blocks/gqa.rs:148-178) and the
gain-free RMS norm (trading_bots/src/torch/model/rmsnorm.rs:16-19).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib as L
from .ssd import _DT, _need, _ptr, _stream, ssd_scan


def _conv_dims(inp, out, width, activation) -> L.SsdConvDims:
    _need(inp.is_cuda and inp.dim() == 3 and inp.dtype in _DT, "conv1d: input must be a CUDA [batch, seqlen, channels] bf16/fp32 tensor")
    _need(inp.stride(2) == 1 and out.stride(2) == 1, "conv1d: the channel dim must be dense")
    d = L.SsdConvDims()
    d.batch, d.seqlen, d.channels = inp.shape
    d.width, d.dtype, d.activation = width, _DT[inp.dtype], 1 if activation else 0
    d.device = inp.device.index if inp.device.index is not None else torch.cuda.current_device()
    d.in_stride_b, d.in_stride_l, d.out_stride_b, d.out_stride_l = inp.stride(0), inp.stride(1), out.stride(0), out.stride(1)
    return d


def conv1d_forward(inp, weight, bias=None, *, activation=True, out=None):
    """out[b,t,c] = act(bias[c] + sum_k weight[c,k] * inp[b,t-K+1+k,c]); weight [C,K] fp32, bias [C] fp32."""
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.dim() == 2, "conv1d: weight must be contiguous fp32 [channels, width]")
    if out is None:
        out = torch.empty_like(inp, memory_format=torch.contiguous_format)
    d = _conv_dims(inp, out, weight.shape[1], activation)
    _need(weight.shape[0] == d.channels, "conv1d: weight rows must equal the channel count")
    with torch.cuda.device(inp.device):
        L.check(L.load().ssd_conv1d_forward(C.byref(d), _ptr(inp), _ptr(weight), _ptr(bias), _ptr(out), _stream(inp.device)))
    return out


def conv1d_backward(inp, weight, bias, douts: Sequence[torch.Tensor], *, activation=True):
    """Gradients of conv1d_forward.  `douts`: the gradient w.r.t. the output as 1-3 tensors [B,L,c_i] whose channel
    counts add up to C (the scan's dx, dB, dC, viewed as [B,L,H*P] / [B,L,G*N]).  Returns din, dweight, dbias."""
    lib = L.load()
    din = torch.empty_like(inp, memory_format=torch.contiguous_format)
    d = _conv_dims(inp, din, weight.shape[1], activation)
    segs = (L.SsdConvGrad * len(douts))()
    for i, g in enumerate(douts):
        _need(g.dim() == 3 and g.dtype == inp.dtype and g.stride(2) == 1 and g.shape[:2] == inp.shape[:2], "conv1d backward: bad gradient segment")
        segs[i].ptr, segs[i].channels, segs[i].stride_b, segs[i].stride_l = g.data_ptr(), g.shape[2], g.stride(0), g.stride(1)
    dweight = torch.empty_like(weight)
    dbias = torch.empty(weight.shape[0], dtype=torch.float32, device=inp.device)
    nbytes = lib.ssd_conv1d_workspace_bytes(C.byref(d))
    _need(nbytes > 0, lib.ssd_last_error().decode())
    ws = torch.empty(nbytes, dtype=torch.uint8, device=inp.device)
    with torch.cuda.device(inp.device):
        L.check(lib.ssd_conv1d_backward(C.byref(d), _ptr(inp), _ptr(weight), _ptr(bias), segs, len(douts), _ptr(din), din.stride(0),
                                        din.stride(1), _ptr(dweight), _ptr(dbias), _ptr(ws), ws.numel(), _stream(inp.device)))
    return din, dweight, dbias


def _norm_dims(inp2, out2, eps) -> L.SsdNormDims:
    d = L.SsdNormDims()
    d.rows, d.width = inp2.shape
    d.dtype, d.eps = _DT[inp2.dtype], eps
    d.device = inp2.device.index if inp2.device.index is not None else torch.cuda.current_device()
    d.in_stride_row, d.out_stride_row = inp2.stride(0), out2.stride(0)
    return d


def rmsnorm_forward(inp, weight=None, *, eps=1e-5):
    """RMS norm over the last dim (all earlier dims are rows).  Returns out, rstd."""
    _need(inp.is_cuda and inp.dtype in _DT and inp.is_contiguous(), "rmsnorm: input must be a contiguous CUDA bf16/fp32 tensor")
    x2 = inp.reshape(-1, inp.shape[-1])
    out = torch.empty_like(x2)
    rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=inp.device)
    d = _norm_dims(x2, out, eps)
    with torch.cuda.device(inp.device):
        L.check(L.load().ssd_rmsnorm_forward(C.byref(d), _ptr(x2), _ptr(weight), _ptr(out), _ptr(rstd), _stream(inp.device)))
    return out.view_as(inp), rstd


def rmsnorm_backward(inp, weight, rstd, dout, *, eps=1e-5):
    """Returns din (shape of inp) and dweight (or None)."""
    lib = L.load()
    x2 = inp.reshape(-1, inp.shape[-1])
    g2 = dout.contiguous().reshape(-1, inp.shape[-1])
    din = torch.empty_like(x2)
    d = _norm_dims(x2, din, eps)
    dweight, ws = None, None
    if weight is not None:
        dweight = torch.empty_like(weight)
        ws = torch.empty(lib.ssd_rmsnorm_workspace_bytes(C.byref(d)), dtype=torch.uint8, device=inp.device)
    with torch.cuda.device(inp.device):
        L.check(lib.ssd_rmsnorm_backward(C.byref(d), _ptr(x2), _ptr(weight), _ptr(rstd), _ptr(g2), g2.stride(0), _ptr(din), din.stride(0),
                                         _ptr(dweight), _ptr(ws), 0 if ws is None else ws.numel(), _stream(inp.device)))
    return din.view_as(inp), dweight


class _Conv1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, weight, bias, activation, splits):
        out = conv1d_forward(inp, weight, bias, activation=activation)
        ctx.save_for_backward(inp, weight, bias)
        ctx.activation, ctx.splits = activation, splits
        return tuple(out.split(splits, dim=2)) if splits else out

    @staticmethod
    def backward(ctx, *gs):
        inp, weight, bias = ctx.saved_tensors
        segs = []
        for g, n in zip(gs, ctx.splits or [inp.shape[2]]):
            if g is None:
                g = torch.zeros(inp.shape[0], inp.shape[1], n, dtype=inp.dtype, device=inp.device)
            g = g.to(inp.dtype)
            segs.append(g if g.stride(2) == 1 and (g.stride(1) * g.element_size()) % 16 == 0 and g.data_ptr() % 16 == 0 else g.contiguous())
        din, dw, db = conv1d_backward(inp, weight, bias, segs, activation=ctx.activation)
        return din, dw, (db if bias is not None else None), None, None


def causal_conv1d(inp, weight, bias=None, *, activation=True, splits: Optional[Sequence[int]] = None):
    """Differentiable causal depthwise conv (+ silu).  With `splits` the output comes back as channel-range views of
    one buffer (what the scan takes as strided x, B, C) and their gradients are consumed as separate segments."""
    return _Conv1d.apply(inp, weight, bias, activation, tuple(splits) if splits else None)


class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, weight, eps):
        out, rstd = rmsnorm_forward(inp, weight, eps=eps)
        ctx.save_for_backward(inp, weight, rstd)
        ctx.eps = eps
        return out

    @staticmethod
    def backward(ctx, g):
        inp, weight, rstd = ctx.saved_tensors
        din, dw = rmsnorm_backward(inp, weight, rstd, g.to(inp.dtype), eps=ctx.eps)
        return din, dw, None


def rmsnorm(inp, weight=None, *, eps=1e-5):
    return _RmsNorm.apply(inp.contiguous(), weight, eps)


def mamba2_mixer_core(xBC, dt, z, conv_weight, conv_bias, dt_bias, A, D, norm_weight, *, nheads, headdim, dstate, ngroups,
                      chunk=128, eps=1e-5, algo="auto", init_state=None):
    """The mixer of a Mamba-2 layer between its two projections, differentiable:
        x, B, C = split(silu(causal_conv1d(xBC)));  y = SSD(x, softplus(dt + dt_bias), A, B, C, D) * silu(z);
        out = rmsnorm(y) * norm_weight.
    xBC [B,L,H*P+2*G*N], dt [B,L,H], z [B,L,H,P].  Four launches of this library's operators: conv, scan (with the
    step-size activation and the gate inside), norm."""
    Bn, Ln, _ = xBC.shape
    hp, gn = nheads * headdim, ngroups * dstate
    x, Bm, Cm = causal_conv1d(xBC, conv_weight, conv_bias, activation=True, splits=(hp, gn, gn))
    y, fin = ssd_scan(x.unflatten(2, (nheads, headdim)), dt, A, Bm.unflatten(2, (ngroups, dstate)),
                      Cm.unflatten(2, (ngroups, dstate)), D, z, init_state, chunk=chunk, algo=algo, dt_bias=dt_bias,
                      dt_softplus=True)
    out = rmsnorm(y.reshape(Bn, Ln, hp), norm_weight, eps=eps)
    return out, fin

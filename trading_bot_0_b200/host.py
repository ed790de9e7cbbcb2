"""Host-buffer entry: forward+backward with every sequence operand in (pinned) host memory.

Batch rows are independent recurrences, so the batch is cut into slices that flow through three
streams: host->device copies of slice i+1, the kernels of slice i and the device->host copies of
slice i-1 overlap, and PCIe (full duplex) rather than the sum of the three sets the pace.  This
is the shape of the reference's rollout boundary, which moves host views in with `from_blob` +
copy and results out once per step (trading_bots/src/torch/train/rollout.rs:67,85-141).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import ssd

_SEQ_IN = ("x", "dt", "B", "C", "dy", "z")
_SEQ_OUT = ("y", "dx", "ddt", "dB", "dC", "dz")


class HostFwdBwd:
    def __init__(self, batch, seqlen, nheads, headdim, dstate, ngroups, chunk, dtype=torch.bfloat16, *, has_z=False,
                 device="cuda:0", slice_batch: Optional[int] = None, slots: int = 3, algo="auto"):
        self.device = torch.device(device)
        self.B, self.L, self.H, self.P, self.N, self.G, self.Q = batch, seqlen, nheads, headdim, dstate, ngroups, chunk
        self.dtype, self.has_z, self.algo = dtype, has_z, algo
        self.sb = slice_batch or max(1, batch // 8)
        self.slots = slots
        dev, sb = self.device, self.sb
        shp = {"x": (sb, seqlen, nheads, headdim), "dt": (sb, seqlen, nheads), "B": (sb, seqlen, ngroups, dstate),
               "C": (sb, seqlen, ngroups, dstate), "dy": (sb, seqlen, nheads, headdim), "z": (sb, seqlen, nheads, headdim)}
        oshp = {"y": shp["x"], "dx": shp["x"], "ddt": shp["dt"], "dB": shp["B"], "dC": shp["B"], "dz": shp["x"]}
        self.inb, self.outb, self.ws = [], [], []
        for _ in range(slots):
            self.inb.append({k: torch.empty(shp[k], dtype=dtype, device=dev) for k in _SEQ_IN if k != "z" or has_z})
            o = {k: torch.empty(oshp[k], dtype=torch.float32 if k == "ddt" else dtype, device=dev)
                 for k in _SEQ_OUT if k != "dz" or has_z}
            o["dA"] = torch.empty(nheads, dtype=torch.float32, device=dev)
            o["dD"] = torch.empty(nheads, dtype=torch.float32, device=dev)
            self.outb.append(o)
            d = ssd.make_dims(self.inb[-1]["x"], self.inb[-1]["dt"], self.inb[-1]["B"], self.inb[-1]["C"], chunk,
                              z=self.inb[-1].get("z"), algo=algo)
            self.ws.append(ssd.alloc_workspace(d, dev, backward=True))
        self.dA = torch.zeros(nheads, dtype=torch.float32, device=dev)
        self.dD = torch.zeros(nheads, dtype=torch.float32, device=dev)
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(slots)]
        self.ev_run = [torch.cuda.Event() for _ in range(slots)]
        self.ev_out = [torch.cuda.Event() for _ in range(slots)]

    def bytes_per_call(self):
        """(host->device, device->host) bytes one call moves, counted from the tensors copied."""
        e = torch.empty(0, dtype=self.dtype).element_size()
        BL = self.B * self.L
        hp, gn = self.H * self.P, self.G * self.N
        h2d = BL * (2 * hp + self.H + 2 * gn + (hp if self.has_z else 0)) * e
        d2h = BL * ((2 * hp + 2 * gn + (hp if self.has_z else 0)) * e + self.H * 4) + 2 * self.H * 4
        return h2d, d2h

    def run(self, host_in: Dict[str, torch.Tensor], A: torch.Tensor, D: torch.Tensor,
            host_out: Dict[str, torch.Tensor]) -> None:
        """host_in: pinned CPU tensors x, dt, B, C, dy (, z) of the full batch; A, D on the device;
        host_out: pinned CPU tensors y, dx, ddt, dB, dC (, dz), dA, dD, filled on return."""
        B, sb = self.B, self.sb
        self.dA.zero_()
        self.dD.zero_()
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        nsl = (B + sb - 1) // sb
        for i in range(nsl):
            k = i % self.slots
            lo, hi = i * sb, min(B, (i + 1) * sb)
            n = hi - lo
            ib, ob = self.inb[k], self.outb[k]
            with torch.cuda.stream(self.s_in):
                if i >= self.slots:
                    self.s_in.wait_event(self.ev_run[k])   # slot's inputs consumed
                for name, buf in ib.items():
                    buf[:n].copy_(host_in[name][lo:hi], non_blocking=True)
                self.ev_in[k].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[k])
                if i >= self.slots:
                    self.s_run.wait_event(self.ev_out[k])  # slot's outputs drained
                z = ib["z"][:n] if self.has_z else None
                ssd.forward(ib["x"][:n], ib["dt"][:n], A, ib["B"][:n], ib["C"][:n], D, z, chunk=self.Q, algo=self.algo,
                            workspace=self.ws[k], y=ob["y"][:n], return_final_state=False)
                out = {"dx": ob["dx"][:n], "ddt": ob["ddt"][:n], "dB": ob["dB"][:n], "dC": ob["dC"][:n],
                       "dA": ob["dA"], "dD": ob["dD"]}
                if self.has_z:
                    out["dz"] = ob["dz"][:n]
                ssd.backward(ib["dy"][:n], ib["x"][:n], ib["dt"][:n], A, ib["B"][:n], ib["C"][:n], D, z, chunk=self.Q,
                             algo=self.algo, workspace=self.ws[k], fwd_saved=True, out=out)
                self.dA += ob["dA"]
                self.dD += ob["dD"]
                self.ev_run[k].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[k])
                for name in _SEQ_OUT:
                    if name in ob:
                        host_out[name][lo:hi].copy_(ob[name][:n], non_blocking=True)
                self.ev_out[k].record(self.s_out)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_stream(self.s_run)
            host_out["dA"].copy_(self.dA, non_blocking=True)
            host_out["dD"].copy_(self.dD, non_blocking=True)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_in)


class HostStep:
    """Streamed-rollout step with the per-step vectors in pinned host memory and the state
    resident on the device: copies x, dt, B, C in, runs the state update, copies y out."""

    def __init__(self, state: torch.Tensor, ngroups: int, dtype=torch.bfloat16):
        S, H, P, N = state.shape
        dev = state.device
        self.state = state
        self.x = torch.empty(S, H, P, dtype=dtype, device=dev)
        self.dt = torch.empty(S, H, dtype=dtype, device=dev)
        self.Bm = torch.empty(S, ngroups, N, dtype=dtype, device=dev)
        self.Cm = torch.empty(S, ngroups, N, dtype=dtype, device=dev)
        self.y = torch.empty(S, H, P, dtype=dtype, device=dev)

    def bytes_per_call(self):
        h2d = sum(t.numel() * t.element_size() for t in (self.x, self.dt, self.Bm, self.Cm))
        return h2d, self.y.numel() * self.y.element_size()

    def step(self, hx, hdt, hB, hC, A, D, hy) -> None:
        self.x.copy_(hx, non_blocking=True)
        self.dt.copy_(hdt, non_blocking=True)
        self.Bm.copy_(hB, non_blocking=True)
        self.Cm.copy_(hC, non_blocking=True)
        ssd.state_update(self.state, self.x, self.dt, A, self.Bm, self.Cm, D, y=self.y)
        hy.copy_(self.y, non_blocking=True)

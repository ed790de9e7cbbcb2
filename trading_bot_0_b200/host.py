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
    """Streamed-rollout step with the per-step vectors in pinned host memory and the state resident on
    the device: one call copies x, dt, B, C in, runs the state update and copies y out.

    The object owns the pinned staging buffers: the caller writes the step's vectors into `hx`, `hdt`,
    `hB`, `hC` (views of ONE packed pinned buffer, one packed row per stream, so a group of streams moves
    with a single copy) and reads the result from `hy`.  The streams (environments) are cut into `groups`
    row ranges that flow through three CUDA streams (host->device copies, kernels, device->host copies),
    the way a rollout double-buffers groups of environments: while one group's kernel runs, the next
    group's inputs arrive and the previous group's outputs leave.  After one eager step the whole step is
    captured into a CUDA graph and replayed, so a step costs one launch on the host
    (trading_bots/src/torch/train/rollout.rs:209-235 is the per-step loop this stands in for).
    `step` returns after enqueueing on the caller's current stream."""

    def __init__(self, state: torch.Tensor, ngroups: int, dtype=torch.bfloat16, groups: int = 8, graph: bool = True):
        S, H, P, N = state.shape
        dev = state.device
        self.state, self.dev = state, dev
        hp, gn = H * P, ngroups * N
        up = lambda n: (n + 7) // 8 * 8                      # every segment of a packed row starts 16-byte aligned
        o_dt, o_b, o_c = up(hp), up(hp) + up(H), up(hp) + up(H) + up(gn)
        self.row = o_c + up(gn)
        self.host_in = torch.zeros(S, self.row, dtype=dtype).pin_memory()
        self.dev_in = torch.zeros(S, self.row, dtype=dtype, device=dev)
        cut = lambda buf: (buf[:, :hp].unflatten(1, (H, P)), buf[:, o_dt:o_dt + H],
                           buf[:, o_b:o_b + gn].unflatten(1, (ngroups, N)),
                           buf[:, o_c:o_c + gn].unflatten(1, (ngroups, N)))
        self.hx, self.hdt, self.hB, self.hC = cut(self.host_in)
        self.x, self.dt, self.Bm, self.Cm = cut(self.dev_in)
        self.y = torch.empty(S, H, P, dtype=dtype, device=dev)
        self.hy = torch.empty(S, H, P, dtype=dtype).pin_memory()
        groups = max(1, min(groups, S))
        per = (S + groups - 1) // groups
        self.ranges = [(lo, min(S, lo + per)) for lo in range(0, S, per)]
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in self.ranges]
        self.ev_run = [torch.cuda.Event() for _ in self.ranges]
        self.use_graph, self._graph, self._calls, self._params = graph, None, 0, None

    def bytes_per_call(self):
        """(host->device, device->host) bytes one step moves, counted from the buffers copied."""
        return self.host_in.numel() * self.host_in.element_size(), self.hy.numel() * self.hy.element_size()

    def load_inputs(self, hx, hdt, hB, hC) -> None:
        """Convenience for callers whose vectors live elsewhere on the host: copy them into the staging views."""
        self.hx.copy_(hx)
        self.hdt.copy_(hdt)
        self.hB.copy_(hB)
        self.hC.copy_(hC)

    def _enqueue(self, root, A, D) -> None:
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(root)
        for gi, (lo, hi) in enumerate(self.ranges):
            with torch.cuda.stream(self.s_in):
                self.dev_in[lo:hi].copy_(self.host_in[lo:hi], non_blocking=True)
                self.ev_in[gi].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[gi])
                ssd.state_update(self.state[lo:hi], self.x[lo:hi], self.dt[lo:hi], A, self.Bm[lo:hi], self.Cm[lo:hi], D,
                                 y=self.y[lo:hi])
                self.ev_run[gi].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[gi])
                self.hy[lo:hi].copy_(self.y[lo:hi], non_blocking=True)
        for s in (self.s_in, self.s_run, self.s_out):
            root.wait_stream(s)

    def step(self, A, D) -> None:
        cur = torch.cuda.current_stream(self.dev)
        self._calls += 1
        if not self.use_graph or self._calls == 1:          # first step eagerly (also warms everything up)
            self._enqueue(cur, A, D)
            return
        key = (A.data_ptr(), D.data_ptr() if D is not None else 0)
        if self._graph is None or self._params != key:
            g = torch.cuda.CUDAGraph()
            cap = torch.cuda.Stream(self.dev)
            cap.wait_stream(cur)
            with torch.cuda.graph(g, stream=cap):
                self._enqueue(cap, A, D)
            cur.wait_stream(cap)
            self._graph, self._params, self._keep = g, key, (A, D)
        self._graph.replay()

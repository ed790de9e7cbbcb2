"""Host-side logic of the sequence-parallel path, run as 2 and 3 gloo ranks on CPU.

The device operations are replaced by the CPU oracle (injected through `ops`), so what is under
test is the slice bookkeeping, the packed all-gather, the direction of both prefix scans, the
boundary-state handling, the dA/dD reduction, and the failure detection of the checked mode: a
rank that never posts, ranks that disagree about the world size or the shapes.  Failures are made
on the host (a rank that skips the call, a wrong argument); nothing here touches a GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ssd_oracle as O
from tests._util import rel_err
from trading_bot_0_b200 import _lib as L
from trading_bot_0_b200 import sp


class OracleOps(sp.SpOps):
    """fp64 CPU stand-in for the CUDA operations behind `sp_forward` / `sp_backward`."""

    def _leaves(self, x, dt, A, Bm, Cm, D, z, init):
        f = lambda t: None if t is None else t.detach().double().requires_grad_(True)
        return [f(t) for t in (x, dt, A, Bm, Cm, D, z, init)]

    def forward(self, stages, x, dt, A, Bm, Cm, D, z, init_state, chunk, algo, workspace, y, final_state):
        if stages & L.STAGE_TOTAL:
            _, total = O.ssd_sequential(x, dt, A, Bm, Cm, D, z, None)
            return None, total.float(), {"ws": True}
        yy, fin = O.ssd_sequential(x, dt, A, Bm, Cm, D, z, init_state)
        return yy, fin.float(), workspace

    def total_logdecay(self, x, dt, A, Bm, Cm, z, chunk, algo, workspace):
        return (dt.double() * A.double()).sum(1).float()

    def prefix_state(self, gs, gl, world, rank, direction, boundary):
        acc = torch.zeros_like(gs[0]) if boundary is None else boundary.clone()
        order = range(rank) if direction > 0 else range(world - 1, rank, -1)
        for q in order:
            acc = torch.exp(gl[q])[..., None, None] * acc + gs[q]
        return acc

    def backward(self, stages, dy, x, dt, A, Bm, Cm, D, z, init_state, dfinal, chunk, algo, workspace, out):
        lv = self._leaves(x, dt, A, Bm, Cm, D, z, init_state)
        yy, fin = O.ssd_sequential(*lv)
        loss = (yy * dy.double()).sum()
        if stages & L.STAGE_FINISH and dfinal is not None:
            loss = loss + (fin * dfinal.double()).sum()
        loss.backward()
        names = ("dx", "ddt", "dA", "dB", "dC", "dD", "dz", "dinit")
        for n, t in zip(names, lv):
            if t is not None:
                out[n] = t.grad.float()
        return out


def _np(t):
    return t.detach().float().cpu().numpy()


def _t(a):
    return torch.from_numpy(a)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        cfg = O.SsdConfig("sp", 2, 96, 2, 4, 8, 1, 16, "fp32", True)
        inp = O.make_inputs(cfg, with_init_state=True)
        dfin = torch.randn(2, 2, 4, 8, generator=torch.Generator().manual_seed(9))
        a, b = sp.slice_bounds(cfg.seqlen, world, rank, cfg.chunk)
        loc = {k: inp[k][:, a:b] for k in ("x", "dt", "B", "C", "z", "dy")}
        ops = OracleOps()
        y, fin, ctx = sp.sp_forward(loc["x"], loc["dt"], inp["A"], loc["B"], loc["C"], inp["D"], loc["z"],
                                    inp["init_state"], chunk=cfg.chunk, ops=ops)
        g = sp.sp_backward(loc["dy"], ctx, dfin, ops=ops)
        # by value (numpy), not as shared-memory handles: a rank may exit before the parent has unpickled its item
        q.put((rank, a, b, _np(y), _np(fin), {k: _np(v) for k, v in g.items() if isinstance(v, torch.Tensor)}))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sp_forward_backward_over_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = sorted([q.get(timeout=90) for _ in range(world)], key=lambda t: t[0])
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    assert all(p.exitcode == 0 for p in procs)
    cfg = O.SsdConfig("sp", 2, 96, 2, 4, 8, 1, 16, "fp32", True)
    inp = O.make_inputs(cfg, with_init_state=True)
    dfin = torch.randn(2, 2, 4, 8, generator=torch.Generator().manual_seed(9))
    ref = O.ssd_grads_autograd(O.ssd_sequential, inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"],
                               inp["dy"], inp["z"], inp["init_state"], dfin)
    assert rel_err(torch.cat([_t(r[3]) for r in res], 1), ref["y"]) < 1e-5
    assert rel_err(_t(res[-1][4]), ref["final_state"]) < 1e-5
    for k in ("dx", "ddt", "dB", "dC", "dz"):
        assert rel_err(torch.cat([_t(r[5][k]) for r in res], 1), ref[k]) < 1e-5, k
    for r in res:  # replicated-parameter gradients are already summed on every rank
        assert rel_err(_t(r[5]["dA"]), ref["dA"]) < 1e-5 and rel_err(_t(r[5]["dD"]), ref["dD"]) < 1e-5
    assert rel_err(_t(res[0][5]["dinit"]), ref["dinit"]) < 1e-5


def test_slice_bounds():
    assert [sp.slice_bounds(1024, 4, r, 128) for r in range(4)] == [(0, 256), (256, 512), (512, 768), (768, 1024)]
    assert sp.slice_bounds(1000, 2, 1, 128) == (512, 1000)
    with pytest.raises(ValueError):
        sp.slice_bounds(128, 4, 3, 128)
    with pytest.raises(ValueError):
        sp.slice_bounds(128, 2, 2, 64)


# ---- failure detection (checked mode) ----------------------------------------------------------------------------
def _spawn(target, world, extra=()):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q) + tuple(extra)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = sorted([q.get(timeout=120) for _ in range(world)], key=lambda t: t[0])
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    assert all(p.exitcode == 0 for p in procs)
    return res


def _slice_inputs(cfg, world, rank):
    inp = O.make_inputs(cfg, with_init_state=True)
    a, b = sp.slice_bounds(cfg.seqlen, world, rank, cfg.chunk)
    return inp, {k: inp[k][:, a:b] for k in ("x", "dt", "B", "C", "dy")}


def _fail_worker(rank, world, port, q, scenario):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        cfg = O.SsdConfig("spf", 1, 64, 2, 4, 8, 1, 16, "fp32", False)
        inp, loc = _slice_inputs(cfg, world, rank)
        ops = OracleOps()
        err = None
        try:
            if scenario == "never_posts":
                if rank != world - 1:      # the last rank skips the exchange altogether
                    sp.sp_forward(loc["x"], loc["dt"], inp["A"], loc["B"], loc["C"], inp["D"], None, None, chunk=cfg.chunk,
                                  ops=ops, timeout_s=1.0, tag="step1")
            elif scenario == "world":
                # one rank believes the job has one rank more than it has
                sig = ("ssd_sp", +1, world + (1 if rank == 0 else 0), 1, 2, 4, 1, 8, cfg.chunk, "torch.float32")
                sp.rendezvous(sig, None, 1.0, "step1")
            elif scenario == "shapes":
                x = loc["x"] if rank != 0 else loc["x"][..., :2]      # rank 0 comes with headdim 2 instead of 4
                sp.sp_forward(x, loc["dt"], inp["A"], loc["B"], loc["C"], inp["D"], None, None, chunk=cfg.chunk, ops=ops,
                              timeout_s=2.0, tag="step1")
        except L.SsdError as e:
            err = (e.code, str(e))
        # the process group is still usable: a collective right after the failure, then a clean checked exchange
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t)
        y, fin, ctx = sp.sp_forward(loc["x"], loc["dt"], inp["A"], loc["B"], loc["C"], inp["D"], None, None, chunk=cfg.chunk,
                                    ops=ops, timeout_s=20.0, tag="retry")
        q.put((rank, err, float(t.item()), _np(y), _np(fin)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("scenario", ["never_posts", "world", "shapes"])
def test_checked_exchange_reports_and_the_group_stays_usable(scenario):
    world = 2
    res = _spawn(_fail_worker, world, (scenario,))
    cfg = O.SsdConfig("spf", 1, 64, 2, 4, 8, 1, 16, "fp32", False)
    inp = O.make_inputs(cfg, with_init_state=True)
    y_ref, fin_ref = O.ssd_sequential(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"])
    errs = {r[0]: r[1] for r in res}
    if scenario == "never_posts":
        assert errs[0] is not None and errs[0][0] == sp.SSD_ERR_TIMEOUT and "[1]" in errs[0][1] and "did not post" in errs[0][1]
        assert errs[1] is None
    else:
        for r in range(world):
            assert errs[r] is not None and errs[r][0] == sp.SSD_ERR_BAD_SHAPE, errs
            assert f"rank {1 - r} posted" in errs[r][1]
    for r in res:
        assert r[2] == 3.0                                   # the all-reduce after the failure
    assert rel_err(torch.cat([_t(r[3]) for r in res], 1), y_ref) < 1e-5      # the clean retry
    assert rel_err(_t(res[-1][4]), fin_ref) < 1e-5

"""The library's own sequence-parallel exchange (NCCL inside the C ABI).  On one GPU: a one-rank communicator through the
raw entry points (unique id, communicator, exchange in both modes, parameter all-reduce) against the plain forward and
backward.  On two GPUs (skipped with fewer): forward/backward split over two ranks against the oracle, for dstate 64 and for
the head shapes of the long-sequence workload."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ssd_oracle as O
from tests._util import assert_close, oracle_all

pytestmark = pytest.mark.gpu
CFGS = {"n64": O.SsdConfig("sp_nccl", 2, 1024, 8, 32, 64, 1, 128, "bf16", False),
        "cfg4_heads": O.SsdConfig("sp_nccl4", 1, 1024, 24, 64, 128, 1, 256, "bf16", False)}


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q, which):
    CFG = CFGS[which]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from trading_bot_0_b200 import sp
        dev = f"cuda:{rank}"
        inp = O.make_inputs(CFG, with_init_state=True)
        dfin = 0.1 * torch.randn(CFG.batch, CFG.nheads, CFG.headdim, CFG.dstate, generator=torch.Generator().manual_seed(9))
        a, b = sp.slice_bounds(CFG.seqlen, world, rank, CFG.chunk)
        loc = {k: inp[k][:, a:b].contiguous().to(dev) for k in ("x", "dt", "B", "C", "dy")}
        A, D, init = inp["A"].to(dev), inp["D"].to(dev), inp["init_state"].to(dev)
        y, fin, ctx = sp.sp_forward(loc["x"], loc["dt"], A, loc["B"], loc["C"], D, None, init, chunk=CFG.chunk,
                                    timeout_s=60.0 if which == "n64" else None)      # one case in checked mode, one unchecked
        g = sp.sp_backward(loc["dy"], ctx, dfin.to(dev))
        from trading_bot_0_b200.ssd import workspace_status
        assert workspace_status(ctx.workspace) == 0
        torch.cuda.synchronize()
        # by value (numpy), not as shared-memory handles: a rank may exit before the parent has unpickled its item
        npy = lambda t: t.detach().float().cpu().numpy()
        q.put((rank, npy(y), npy(fin), {k: npy(v) for k, v in g.items() if isinstance(v, torch.Tensor) and k != "workspace"}))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("which", ["n64", "cfg4_heads"])
def test_sequence_parallel_over_nccl_matches_oracle(lib, which):
    world = 2
    CFG = CFGS[which]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, which)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = sorted([q.get(timeout=240) for _ in range(world)], key=lambda t: t[0])
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    assert all(p.exitcode == 0 for p in procs)
    res = [(r[0], torch.from_numpy(r[1]), torch.from_numpy(r[2]), {k: torch.from_numpy(v) for k, v in r[3].items()}) for r in res]
    inp = O.make_inputs(CFG, with_init_state=True)
    dfin = 0.1 * torch.randn(CFG.batch, CFG.nheads, CFG.headdim, CFG.dstate, generator=torch.Generator().manual_seed(9))
    ref = oracle_all(inp, dfin)
    assert_close("y", torch.cat([r[1] for r in res], 1), ref["y"], "bf16")
    assert_close("final_state", res[-1][2], ref["final_state"], "bf16")
    for k in ("dx", "ddt", "dB", "dC"):
        assert_close(k, torch.cat([r[3][k] for r in res], 1), ref[k], "bf16")
    for r in res:
        assert_close("dA", r[3]["dA"], ref["dA"], "bf16")
        assert_close("dD", r[3]["dD"], ref["dD"], "bf16")
    assert_close("dinit", res[0][3]["dinit"], ref["dinit"], "bf16")


def test_library_exchange_with_a_one_rank_communicator(lib):
    """The raw entry points a host without torch.distributed would call: NCCL id, communicator, LOCAL|TOTAL -> exchange ->
    FINISH forward, the mirrored backward, the parameter all-reduce; unchecked (timeout 0) and checked (signature round +
    bounded host wait).  With one rank the exchange must hand back the boundary state itself, so the staged result has to
    equal the plain forward / backward bit for bit where the same kernels run, and the oracle within the bf16 gate."""
    import ctypes as C
    import trading_bot_0_b200 as T
    from trading_bot_0_b200 import _lib as L
    from trading_bot_0_b200.ssd import _ptr, make_dims, workspace_status
    dev = torch.device("cuda:0")
    cfg = O.SsdConfig("sp_one", 2, 512, 24, 64, 128, 1, 256, "bf16", False)
    inp = O.make_inputs(cfg, with_init_state=True)
    dfin = 0.1 * torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.dstate, generator=torch.Generator().manual_seed(9))
    ref = oracle_all(inp, dfin)
    d = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in inp.items()}
    ident = (C.c_ubyte * L.SP_UNIQUE_ID_BYTES)()
    with torch.cuda.device(dev):
        assert lib.ssd_sp_unique_id(ident) == 0, lib.ssd_last_error().decode()
        comm = lib.ssd_sp_comm_new(ident, 1, 0)
    assert comm, lib.ssd_last_error().decode()
    try:
        assert lib.ssd_sp_comm_world(comm) == 1 and lib.ssd_sp_comm_rank(comm) == 0
        args = (d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], None)
        dims = make_dims(d["x"], d["dt"], d["B"], d["C"], cfg.chunk)
        nb = lib.ssd_sp_exchange_bytes(C.byref(dims), 1)
        assert nb > 0
        exch = torch.empty(nb, dtype=torch.uint8, device=dev)
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        for timeout_ms in (0, 5000):
            y, total, ws = T.forward(*args, None, chunk=cfg.chunk, for_backward=True, stages=L.STAGE_LOCAL | L.STAGE_TOTAL)
            state_in = torch.empty_like(total)
            with torch.cuda.device(dev):
                rc = lib.ssd_sp_exchange_fwd(C.byref(dims), _ptr(ws), ws.numel(), comm, _ptr(total), _ptr(d["init_state"]),
                                             _ptr(state_in), _ptr(exch), nb, stream, timeout_ms)
            assert rc == 0, lib.ssd_last_error().decode()
            torch.cuda.synchronize()
            assert torch.equal(state_in, d["init_state"])
            y, fin, ws = T.forward(*args, state_in, chunk=cfg.chunk, workspace=ws, y=y, final_state=total, stages=L.STAGE_FINISH)
            assert_close("y", y, ref["y"], "bf16")
            assert_close("final_state", fin, ref["final_state"], "bf16")
            out = {}
            g = T.backward(d["dy"], *args, state_in, None, chunk=cfg.chunk, workspace=ws, fwd_saved=True, want_dinit=True,
                           stages=L.STAGE_LOCAL_STATES | L.STAGE_TOTAL, out=out)
            dstate_out = torch.empty_like(total)
            dfin_d = dfin.to(dev)
            with torch.cuda.device(dev):
                rc = lib.ssd_sp_exchange_bwd(C.byref(dims), _ptr(ws), ws.numel(), comm, _ptr(g["dinit"]), _ptr(dfin_d),
                                             _ptr(dstate_out), _ptr(exch), nb, stream, timeout_ms)
            assert rc == 0, lib.ssd_last_error().decode()
            T.backward(d["dy"], *args, state_in, None, chunk=cfg.chunk, workspace=ws, fwd_saved=True, want_dinit=True,
                       stages=L.STAGE_LOCAL_REST, out=out)
            g = T.backward(d["dy"], *args, state_in, dstate_out, chunk=cfg.chunk, workspace=ws, fwd_saved=True, want_dinit=True,
                           stages=L.STAGE_FINISH, out=out)
            with torch.cuda.device(dev):
                assert lib.ssd_sp_allreduce_params(comm, _ptr(g["dA"]), _ptr(g["dD"]), cfg.nheads, stream, timeout_ms) == 0
            assert workspace_status(ws) == 0
            assert torch.equal(dstate_out, dfin_d)
            for k in ("dx", "ddt", "dA", "dB", "dC", "dD", "dinit"):
                assert_close(k, g[k], ref[k], "bf16")
        # a too-small exchange buffer and a NULL communicator are error codes
        with torch.cuda.device(dev):
            assert lib.ssd_sp_exchange_fwd(C.byref(dims), _ptr(ws), ws.numel(), comm, _ptr(total), None, _ptr(state_in),
                                           _ptr(exch), 256, stream, 0) == -4
            assert lib.ssd_sp_exchange_fwd(C.byref(dims), _ptr(ws), ws.numel(), None, _ptr(total), None, _ptr(state_in),
                                           _ptr(exch), nb, stream, 0) == -6
    finally:
        lib.ssd_sp_comm_free(comm)

"""Sequence-parallel forward/backward over NCCL on 2 real GPUs against the unsplit result on one.
Skipped when the box has fewer than 2 GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ssd_oracle as O
from tests._util import assert_close, oracle_all

pytestmark = pytest.mark.gpu
CFG = O.SsdConfig("sp_nccl", 2, 1024, 8, 32, 64, 1, 128, "bf16", False)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
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
        y, fin, ctx = sp.sp_forward(loc["x"], loc["dt"], A, loc["B"], loc["C"], D, None, init, chunk=CFG.chunk)
        g = sp.sp_backward(loc["dy"], ctx, dfin.to(dev))
        torch.cuda.synchronize()
        q.put((rank, y.cpu(), fin.cpu(), {k: v.cpu() for k, v in g.items() if isinstance(v, torch.Tensor) and k != "workspace"}))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sequence_parallel_over_nccl_matches_oracle(lib):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
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

"""The libtorch autograd node (csrc/ssd_torch.cpp): the C++ caller program that goes through the libtch-style C entry
points, and the same node reached from Python as torch.ops.ssd_b200.*."""
import subprocess

import pytest
import torch

from oracle import ssd_oracle as O
from tests._util import assert_close, cfg_like, oracle_all, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_cpp_caller_through_the_c_entry_points(lib):
    """Parity with the defining recurrence (fp64, libtorch autograd on the CPU), CUDA-graph capture of forward + backward on
    a side stream, the single-step entry point and error reporting, all in C++ (tests/cpp/ssd_torch_caller.cpp)."""
    from trading_bot_0_b200 import build as B
    assert B.CALLER.exists(), f"{B.CALLER} is missing: run `python -m trading_bot_0_b200.build --torch`"
    r = subprocess.run([str(B.CALLER)], capture_output=True, text=True, timeout=600)
    print(r.stdout[-4000:], r.stderr[-2000:])
    assert r.returncode == 0 and "ALL OK" in r.stdout


@pytest.mark.parametrize("base,kw", [(0, dict(has_z=True)), (1, dict(batch=2, seqlen=384)), (1, dict(batch=3, seqlen=384, has_z=True))])
def test_node_matches_oracle_and_python_autograd(lib, base, kw):
    import trading_bot_0_b200 as T
    from trading_bot_0_b200 import torch_node as TN
    cfg = cfg_like(base, **kw)
    inp = O.make_inputs(cfg, with_init_state=True)
    dfin = 0.1 * torch.randn(inp["init_state"].shape, generator=torch.Generator().manual_seed(5))   # at the state's own magnitude
    ref = oracle_all(inp, dfin)
    names = ("x", "dt", "A", "B", "C", "D", "z", "init_state")

    def run(fn):
        d = to_dev(inp, DEV)
        leaves = [d[k].clone().requires_grad_(True) if d.get(k) is not None else None for k in names]
        y, fin = fn(*leaves, chunk=cfg.chunk)
        ((y.float() * d["dy"].float()).sum() + (fin * dfin.to(DEV)).sum()).backward()
        return y, fin, [None if v is None else v.grad for v in leaves]

    y, fin, grads = run(TN.ssd_scan)
    y2, fin2, grads2 = run(T.ssd_scan)
    assert_close("y", y, ref["y"], cfg.dtype)
    assert_close("final_state", fin, ref["final_state"], cfg.dtype)
    for k, g, g2 in zip(("dx", "ddt", "dA", "dB", "dC", "dD", "dz", "dinit"), grads, grads2):
        if g is None:
            continue
        assert_close(k, g, ref[k], cfg.dtype)
        assert torch.equal(g, g2), f"{k}: the C++ node and the Python autograd function run the same kernels"
    assert torch.equal(y, y2) and torch.equal(fin, fin2)


def test_node_forward_only_and_step(lib):
    """No input requires a gradient: the node takes the smaller forward workspace; the step operator updates in place."""
    from trading_bot_0_b200 import torch_node as TN
    import trading_bot_0_b200 as T
    cfg = cfg_like(1, batch=2, seqlen=256)
    d = to_dev(O.make_inputs(cfg), DEV)
    with torch.no_grad():
        y, fin = TN.ssd_scan(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=cfg.chunk)
    y2, fin2, _ = T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=cfg.chunk)
    assert torch.equal(y, y2) and torch.equal(fin, fin2) and not y.requires_grad
    dec = to_dev(O.make_decode_inputs(cfg_like(2, batch=32), 2), DEV)
    s1, s2 = dec["state"].clone(), dec["state"].clone()
    for t in range(2):
        ya = TN.state_update(s1, dec["x"][t], dec["dt"][t], dec["A"], dec["B"][t], dec["C"][t], dec["D"])
        yb = T.state_update(s2, dec["x"][t], dec["dt"][t], dec["A"], dec["B"][t], dec["C"][t], dec["D"])
    assert torch.equal(ya, yb) and torch.equal(s1, s2)


def test_node_rejects_bad_input(lib):
    from trading_bot_0_b200 import torch_node as TN
    cfg = cfg_like(1, batch=1, seqlen=128)
    d = to_dev(O.make_inputs(cfg), DEV)
    with pytest.raises(RuntimeError, match="dt must have shape"):
        TN.ssd_scan(d["x"], d["dt"][:, :64], d["A"], d["B"], d["C"], chunk=cfg.chunk)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        TN.ssd_scan(d["x"].cpu(), d["dt"].cpu(), d["A"].cpu(), d["B"].cpu(), d["C"].cpu(), chunk=cfg.chunk)

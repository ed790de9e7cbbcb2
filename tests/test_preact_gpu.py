"""Step-size pre-activation fused into the operator: dt = act(dt_raw + dt_bias), forward, backward and rollout step."""
import pytest
import torch

from oracle import ssd_oracle as O
from tests._util import assert_close, oracle_all, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _raw_inputs(cfg, softplus):
    """cfg's draws, except that `dt` holds the raw value before bias and activation."""
    inp = O.make_inputs(cfg, with_init_state=True)
    g = torch.Generator().manual_seed(11)
    H = cfg.nheads
    dt0 = torch.exp(torch.log(torch.tensor(1e-3)) + torch.rand(H, generator=g) * torch.log(torch.tensor(100.0)))
    bias = dt0 + torch.log(-torch.expm1(-dt0)) if softplus else 0.5 * dt0
    raw = 0.5 * torch.randn(cfg.batch, cfg.seqlen, H, generator=g)
    if not softplus:
        raw = raw.abs() * 0.05 + 0.005          # identity activation: keep the step size positive
    inp["dt_raw"] = raw.to(O.torch_dtype(cfg.dtype))
    inp["dt_bias"] = bias.float()
    return inp


def _reference(inp, softplus, dfinal=None):
    dt_eff, dact = O.dt_preactivation(inp["dt_raw"], inp["dt_bias"], softplus)
    ref = oracle_all(dict(inp, dt=dt_eff), dfinal)
    ref["ddt_raw"] = ref["ddt"].double() * dact
    ref["ddt_bias"] = ref["ddt_raw"].sum(dim=(0, 1))
    return ref


@pytest.mark.parametrize("softplus", [True, False])
@pytest.mark.parametrize("dtype,algo,dims", [("fp32", "fp32_cores", (4, 256, 4, 32, 16, 1, 64)),
                                             ("bf16", "tensor", (3, 384, 8, 32, 64, 1, 128)),
                                             ("bf16", "tensor", (2, 256, 4, 64, 128, 2, 128))])
def test_fused_preactivation_forward_backward(lib, dtype, algo, dims, softplus):
    import trading_bot_0_b200 as T
    Bn, L, H, P, N, G, Q = dims
    cfg = O.SsdConfig("pre", Bn, L, H, P, N, G, Q, dtype, False)
    inp = _raw_inputs(cfg, softplus)
    dfinal = 0.1 * torch.randn(Bn, H, P, N, generator=torch.Generator().manual_seed(4))
    ref = _reference(inp, softplus, dfinal)
    d = to_dev(inp, DEV)
    y, fin, ws = T.forward(d["x"], d["dt_raw"], d["A"], d["B"], d["C"], d["D"], None, d["init_state"], chunk=Q, algo=algo,
                           for_backward=True, dt_bias=d["dt_bias"], dt_softplus=softplus)
    assert_close("y", y, ref["y"], dtype)
    assert_close("final_state", fin, ref["final_state"], dtype)
    g = T.backward(d["dy"], d["x"], d["dt_raw"], d["A"], d["B"], d["C"], d["D"], None, d["init_state"], dfinal.to(DEV),
                   chunk=Q, algo=algo, workspace=ws, fwd_saved=True, dt_bias=d["dt_bias"], dt_softplus=softplus)
    for k in ("dx", "dA", "dB", "dC", "dD", "dinit"):
        assert_close(k, g[k], ref[k], dtype)
    assert_close("ddt (raw)", g["ddt"], ref["ddt_raw"], dtype)
    assert_close("ddt_bias", g["ddt_bias"], ref["ddt_bias"], dtype)
    # the same without the saved forward state (everything recomputed from the raw inputs)
    g2 = T.backward(d["dy"], d["x"], d["dt_raw"], d["A"], d["B"], d["C"], d["D"], None, d["init_state"], dfinal.to(DEV),
                    chunk=Q, algo=algo, dt_bias=d["dt_bias"], dt_softplus=softplus)
    assert_close("ddt (raw, recomputed)", g2["ddt"], ref["ddt_raw"], dtype)
    assert_close("ddt_bias (recomputed)", g2["ddt_bias"], ref["ddt_bias"], dtype)


def test_fused_preactivation_rollout_step(lib):
    import trading_bot_0_b200 as T
    cfg = O.SsdConfig("dec", 33, 1, 8, 32, 64, 1, 1, "bf16")
    steps = 5
    inp = O.make_decode_inputs(cfg, steps)
    g = torch.Generator().manual_seed(5)
    raw = (0.5 * torch.randn(steps, 33, 8, generator=g)).bfloat16()
    bias = torch.randn(8, generator=g) - 3.0
    dt_eff, _ = O.dt_preactivation(raw, bias, True)
    S = inp["state"].double()
    ys = []
    for t in range(steps):
        y, S = O.state_update(S, inp["x"][t], dt_eff[t], inp["A"], inp["B"][t], inp["C"][t], inp["D"])
        ys.append(y)
    d = to_dev(inp, DEV)
    st = d["state"].clone()
    got = [T.state_update(st, d["x"][t], raw[t].to(DEV), d["A"], d["B"][t], d["C"][t], d["D"], dt_bias=bias.to(DEV),
                          dt_softplus=True) for t in range(steps)]
    assert_close("y", torch.stack(got), torch.stack(ys), "bf16")
    assert_close("state", st, S, "bf16")


def test_autograd_function_with_bias(lib):
    import trading_bot_0_b200 as T
    cfg = O.SsdConfig("pre", 2, 256, 8, 32, 64, 1, 128, "bf16", False)
    inp = _raw_inputs(cfg, True)
    ref = _reference(inp, True)
    d = to_dev(inp, DEV)
    x = d["x"].clone().requires_grad_(True)
    dtr = d["dt_raw"].clone().requires_grad_(True)
    bias = d["dt_bias"].clone().requires_grad_(True)
    y, _ = T.ssd_scan(x, dtr, d["A"], d["B"], d["C"], d["D"], None, d["init_state"], chunk=128, dt_bias=bias, dt_softplus=True)
    (y.float() * d["dy"].float()).sum().backward()
    assert_close("dx", x.grad, ref["dx"], "bf16")
    assert_close("ddt_bias", bias.grad, ref["ddt_bias"], "bf16")
    assert_close("ddt (raw)", dtr.grad, ref["ddt_raw"], "bf16")

"""Streamed-rollout step: parity with the oracle recurrence, prefill/step equivalence, reset."""
import pytest
import torch

from oracle import ssd_oracle as O
from tests._util import assert_close, cfg_like, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def oracle_steps(inp, steps, z=None):
    S = inp["state"].double()
    ys = []
    for t in range(steps):
        y, S = O.state_update(S, inp["x"][t], inp["dt"][t], inp["A"], inp["B"][t], inp["C"][t], inp["D"],
                              None if z is None else z[t])
        ys.append(y)
    return torch.stack(ys), S


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("H,P,N,G", [(8, 32, 64, 1), (4, 32, 16, 1), (24, 64, 128, 1), (2, 16, 256, 2),
                                     (6, 24, 40, 3), (4, 20, 32, 2)])
def test_state_update_matches_oracle(lib, dtype, H, P, N, G):
    import trading_bot_0_b200 as T
    cfg = O.SsdConfig("dec", 33, 1, H, P, N, G, 1, dtype)
    steps = 12
    inp = O.make_decode_inputs(cfg, steps)
    z = torch.randn(steps, 33, H, P, generator=torch.Generator().manual_seed(3)).to(O.torch_dtype(dtype))
    ref_y, ref_S = oracle_steps(inp, steps, z)
    d = to_dev(inp, DEV)
    zd = z.to(DEV)
    st = T.StreamState(d["state"].clone())
    ys = [st.step(d["x"][t], d["dt"][t], d["A"], d["B"][t], d["C"][t], d["D"], zd[t]) for t in range(steps)]
    assert_close("y", torch.stack(ys), ref_y, dtype)
    assert_close("state", st.state, ref_S, "fp32" if dtype == "fp32" else "bf16")


def test_prefill_then_steps_equals_full(lib):
    """chunk-scan over the first k tokens, then L-k single steps, equals the chunk-scan over all L
    (the SSD analogue of `cached_forward_matches_full_forward`,
    trading_bots/src/torch/world_model.rs:2683-2718: prefill 32, then 32 steps, max-abs < 1e-4)."""
    import trading_bot_0_b200 as T
    cfg = cfg_like(0, seqlen=64, chunk=32)
    d = to_dev(O.make_inputs(cfg), DEV)
    y_full, fin_full, _ = T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=cfg.chunk)
    k = 32
    y_pre, fin, _ = T.forward(d["x"][:, :k], d["dt"][:, :k], d["A"], d["B"][:, :k], d["C"][:, :k], d["D"],
                              chunk=cfg.chunk)
    st = T.StreamState(fin)
    ys = [y_pre]
    for t in range(k, cfg.seqlen):
        ys.append(st.step(d["x"][:, t], d["dt"][:, t], d["A"], d["B"][:, t], d["C"][:, t], d["D"])[:, None])
    y_cat = torch.cat(ys, 1)
    assert (y_cat - y_full).abs().max().item() < 1e-4
    assert (st.state - fin_full).abs().max().item() < 1e-4


def test_batched_equals_per_stream(lib):
    """Batched step == each stream stepped alone (mirror of the windowed-replay-vs-sequential test,
    trading_bots/src/torch/model/stream/replay.rs:263-353)."""
    import trading_bot_0_b200 as T
    cfg = cfg_like(2, batch=5, dtype="fp32")
    d = to_dev(O.make_decode_inputs(cfg, 3), DEV)
    st = T.StreamState(d["state"].clone())
    singles = [T.StreamState(d["state"][s:s + 1].clone()) for s in range(5)]
    for t in range(3):
        y = st.step(d["x"][t], d["dt"][t], d["A"], d["B"][t], d["C"][t], d["D"])
        for s in range(5):
            ys = singles[s].step(d["x"][t, s:s + 1], d["dt"][t, s:s + 1], d["A"], d["B"][t, s:s + 1],
                                 d["C"][t, s:s + 1], d["D"])
            assert torch.equal(ys[0], y[s])
    for s in range(5):
        assert torch.equal(singles[s].state[0], st.state[s])


def test_mid_rollout_stream_reset(lib):
    """Zeroing selected streams between steps == restarting those streams from a zero state
    (mirror of the mid-chunk env reset test, trading_bots/src/torch/model/stream/replay.rs:360-485)."""
    import trading_bot_0_b200 as T
    cfg = cfg_like(2, batch=9, dtype="fp32")
    d = to_dev(O.make_decode_inputs(cfg, 4), DEV)
    st = T.StreamState(d["state"].clone())
    fresh = T.init_stream_state_batched(9, cfg.nheads, cfg.headdim, cfg.dstate, DEV)
    idx = torch.tensor([1, 4, 8], device=DEV)
    for t in range(2):
        st.step(d["x"][t], d["dt"][t], d["A"], d["B"][t], d["C"][t], d["D"])
    st.reset_streams(idx)
    assert st.state[idx].abs().max().item() == 0.0 and st.state[0].abs().max().item() > 0.0
    for t in range(2, 4):
        y = st.step(d["x"][t], d["dt"][t], d["A"], d["B"][t], d["C"][t], d["D"])
        yf = fresh.step(d["x"][t], d["dt"][t], d["A"], d["B"][t], d["C"][t], d["D"])
    assert torch.equal(y[idx], yf[idx])
    st.reset()
    assert st.state.abs().max().item() == 0.0


@pytest.mark.parametrize("groups,graph", [(1, False), (3, True), (8, True)])
def test_host_step_groups_match_oracle(lib, groups, graph):
    """The host-buffer rollout step (pinned staging buffers, streams cut into row groups that overlap on three CUDA
    streams, the step replayed from a CUDA graph) gives the oracle's outputs and state, whatever the number of groups
    (33 streams: ragged last group)."""
    from trading_bot_0_b200.host import HostStep
    cfg = O.SsdConfig("dec", 33, 1, 8, 32, 64, 1, 1, "bf16")
    steps = 6
    inp = O.make_decode_inputs(cfg, steps)
    ref_y, ref_S = oracle_steps(inp, steps)
    d = to_dev(inp, DEV)
    state = d["state"].clone()
    hs = HostStep(state, cfg.ngroups, groups=groups, graph=graph)
    ys = []
    for t in range(steps):
        hs.load_inputs(inp["x"][t], inp["dt"][t], inp["B"][t], inp["C"][t])
        hs.step(d["A"], d["D"])
        torch.cuda.synchronize()
        ys.append(hs.hy.clone())
    assert_close("y", torch.stack(ys).to(DEV), ref_y, "bf16")
    assert_close("state", state, ref_S, "bf16")

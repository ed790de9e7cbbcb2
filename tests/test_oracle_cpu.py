"""The CPU oracle checked against itself and against the committed fixtures (no GPU)."""
import dataclasses
import os

import numpy as np
import pytest
import torch

from oracle import ssd_oracle as O
from tests._util import rel_err

GOLD = os.path.join(os.path.dirname(__file__), "golden", "ssd_small.npz")


def _inputs(has_z=True):
    cfg = dataclasses.replace(O.CONFIGS[0], batch=2, seqlen=128, has_z=has_z)
    return cfg, O.make_inputs(cfg, with_init_state=True)


@pytest.mark.parametrize("has_z", [False, True])
def test_manual_reverse_recurrence_matches_autograd(has_z):
    cfg, inp = _inputs(has_z)
    dfin = torch.randn(2, cfg.nheads, cfg.headdim, cfg.dstate, generator=torch.Generator().manual_seed(1))
    a = O.ssd_grads_autograd(O.ssd_sequential, inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], inp["dy"],
                             inp.get("z"), inp["init_state"], dfin)
    m = O.ssd_sequential_grads_manual(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], inp["dy"],
                                      inp.get("z"), inp["init_state"], dfin)
    for k, v in a.items():
        assert rel_err(torch.from_numpy(np.asarray(m[k])), v) < 1e-12, k


@pytest.mark.parametrize("chunk", [16, 32, 64, 128])
def test_chunked_equals_sequential_for_every_chunk(chunk):
    cfg, inp = _inputs()
    s = O.ssd_grads_autograd(O.ssd_sequential, inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], inp["dy"],
                             inp["z"], inp["init_state"])
    c = O.ssd_grads_autograd(O.ssd_chunked, inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], inp["dy"],
                             inp["z"], inp["init_state"], dtype=torch.float64, chunk=chunk)
    for k, v in s.items():
        assert rel_err(c[k], v) < 1e-10, k


def test_chunked_fp32_is_within_the_fp32_gate():
    cfg, inp = _inputs()
    s = O.ssd_grads_autograd(O.ssd_sequential, inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], inp["dy"],
                             inp["z"], inp["init_state"])
    c = O.ssd_grads_autograd(O.ssd_chunked, inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], inp["dy"],
                             inp["z"], inp["init_state"], dtype=torch.float32, chunk=64)
    for k, v in s.items():
        assert rel_err(c[k], v) < 1e-4, k


def test_prefill_then_steps_equals_full():
    cfg, inp = _inputs(False)
    y, S = O.ssd_sequential(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"])
    k = 64
    yp, Sp = O.ssd_chunked(inp["x"][:, :k], inp["dt"][:, :k], inp["A"], inp["B"][:, :k], inp["C"][:, :k], inp["D"],
                           chunk=32, dtype=torch.float64)
    ys = [yp]
    for t in range(k, cfg.seqlen):
        yt, Sp = O.state_update(Sp, inp["x"][:, t], inp["dt"][:, t], inp["A"], inp["B"][:, t], inp["C"][:, t], inp["D"])
        ys.append(yt[:, None])
    assert rel_err(torch.cat(ys, 1), y) < 1e-12 and rel_err(Sp, S) < 1e-12


def test_input_distributions():
    inp = O.make_inputs(O.CONFIGS[0])
    assert inp["x"].shape == (4, 256, 4, 32) and inp["B"].shape == (4, 256, 1, 16)
    assert (inp["dt"] > 0).all() and (inp["A"] <= -1).all() and (inp["A"] >= -16).all()
    assert abs(float(inp["x"].std()) - 1.0) < 0.02
    assert abs(float(inp["B"].std()) - 0.25) < 0.01
    assert torch.equal(inp["D"], torch.ones(4))
    bf = O.make_inputs(dataclasses.replace(O.CONFIGS[1], batch=1, seqlen=8))
    assert bf["x"].dtype == torch.bfloat16 and bf["A"].dtype == torch.float32


def test_golden_fixture_reproduces():
    from tests.golden.make_golden import CFG, SEED
    g = np.load(GOLD)
    inp = O.make_inputs(CFG, SEED, with_init_state=True)
    for k, v in inp.items():
        assert np.array_equal(g["in_" + k], v.numpy()), k
    dfin = torch.from_numpy(g["in_dfinal"])
    a = O.ssd_grads_autograd(O.ssd_chunked, inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], inp["dy"],
                             inp["z"], inp["init_state"], dfin, dtype=torch.float64, chunk=CFG.chunk)
    for k, v in a.items():
        assert rel_err(v, torch.from_numpy(g["ref_" + k])) < 1e-10, k


def test_prepost_references_match_torch_ops():
    """The conv / norm / step-size references restate torch's own operators (fp64)."""
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(2)
    x = torch.randn(2, 19, 16, generator=g, dtype=torch.float64)
    w = torch.randn(16, 4, generator=g, dtype=torch.float64)
    b = torch.randn(16, generator=g, dtype=torch.float64)
    want = F.silu(F.conv1d(F.pad(x.transpose(1, 2), (3, 0)), w[:, None, :], b, groups=16).transpose(1, 2))
    assert (O.causal_conv1d_ref(x, w, b, True) - want).abs().max() < 1e-12
    n = O.rmsnorm_ref(x, b, 1e-5)
    assert (n - F.rms_norm(x, (16,), b, 1e-5)).abs().max() < 1e-12
    raw = torch.randn(3, 5, 4, generator=g, dtype=torch.float64).requires_grad_(True)
    bias = torch.randn(4, generator=g, dtype=torch.float64)
    dt, dact = O.dt_preactivation(raw, bias, True)
    dt.sum().backward()
    assert (raw.grad - dact).abs().max() < 1e-12
    assert (dt - F.softplus(raw + bias)).abs().max() < 1e-12

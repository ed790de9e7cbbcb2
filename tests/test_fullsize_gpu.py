"""Size-independent properties checked at the full workload sizes (where the CPU oracle would take
minutes): the operator is linear in x, in B and in C separately, so forward and backward must be
adjoint; a sequence may be cut anywhere and resumed from the carried state; batch rows are
independent; chunk-scan prefill followed by single steps equals the full chunk-scan."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CFGS = {
    "cfg1": dict(B=512, L=1024, H=8, P=32, N=64, G=1, Q=128, z=False),
    "cfg3": dict(B=16, L=4096, H=24, P=64, N=128, G=1, Q=256, z=True),
    "cfg4_one_gpu": dict(B=2, L=131072, H=24, P=64, N=128, G=1, Q=256, z=False),
}


def draw(c, seed=20260811, L=None):
    g = torch.Generator(device=DEV).manual_seed(seed)
    B, L, H, P, N, G = c["B"], L or c["L"], c["H"], c["P"], c["N"], c["G"]
    r = lambda *s: torch.randn(*s, generator=g, device=DEV)
    u = torch.rand(H, generator=g, device=DEV)
    dt0 = torch.exp(math.log(1e-3) + u * math.log(100.0))
    dt_bias = dt0 + torch.log(-torch.expm1(-dt0))
    out = dict(x=r(B, L, H, P).bfloat16(), dt=F.softplus(0.5 * r(B, L, H) + dt_bias).bfloat16(),
               A=-torch.exp(torch.rand(H, generator=g, device=DEV) * math.log(16.0)),
               B=(r(B, L, G, N) / math.sqrt(N)).bfloat16(), C=(r(B, L, G, N) / math.sqrt(N)).bfloat16(),
               D=torch.ones(H, device=DEV), dy=r(B, L, H, P).bfloat16())
    if c["z"]:
        out["z"] = r(B, L, H, P).bfloat16()
    return out


def rel(a, b):
    return float((a.double() - b.double()).abs().max() / (b.double().abs().max() + 1e-30))


@pytest.mark.parametrize("name", ["cfg1", "cfg3", "cfg4_one_gpu"])
def test_forward_backward_are_adjoint(lib, name):
    """<dy, F(v)> == <F^T(dy), v> for the maps x -> y, B -> y and C -> y (ungated, D = 0, so each
    map is exactly linear); bf16 outputs bound the agreement to about 1e-2."""
    import trading_bot_0_b200 as T
    c = CFGS[name]
    d = draw(c)
    g = T.backward(d["dy"], d["x"], d["dt"], d["A"], d["B"], d["C"], None, None, chunk=c["Q"])
    y, _, _ = T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], None, None, chunk=c["Q"])
    lhs = float((d["dy"].double() * y.double()).sum())
    for key, grad in (("x", "dx"), ("B", "dB"), ("C", "dC")):
        rhs = float((g[grad].double() * d[key].double()).sum())
        assert abs(lhs - rhs) <= 1e-2 * max(abs(lhs), abs(rhs)) + 1e-3 * math.sqrt(y.numel()), (name, key, lhs, rhs)


@pytest.mark.parametrize("name", ["cfg1", "cfg3", "cfg4_one_gpu"])
def test_cut_and_resume_from_carried_state(lib, name):
    import trading_bot_0_b200 as T
    c = CFGS[name]
    d = draw(c)
    z = d.get("z")
    y, fin, _ = T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], z, chunk=c["Q"])
    k = c["L"] // 2
    cut = lambda t, a, b: None if t is None else t[:, a:b]
    y1, s1, _ = T.forward(cut(d["x"], 0, k), cut(d["dt"], 0, k), d["A"], cut(d["B"], 0, k), cut(d["C"], 0, k), d["D"],
                          cut(z, 0, k), chunk=c["Q"])
    y2, s2, _ = T.forward(cut(d["x"], k, None), cut(d["dt"], k, None), d["A"], cut(d["B"], k, None),
                          cut(d["C"], k, None), d["D"], cut(z, k, None), s1, chunk=c["Q"])
    assert torch.equal(y[:, :k], y1)
    assert (y[:, k:].float() - y2.float()).abs().max().item() <= 2e-2
    assert rel(s2, fin) <= 1e-3


def test_batch_rows_are_independent(lib):
    import trading_bot_0_b200 as T
    c = CFGS["cfg1"]
    d = draw(c)
    y, fin, _ = T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=c["Q"])
    sl = slice(100, 108)
    ys, fs, _ = T.forward(d["x"][sl], d["dt"][sl], d["A"], d["B"][sl], d["C"][sl], d["D"], chunk=c["Q"])
    assert torch.equal(y[sl], ys) and torch.equal(fin[sl], fs)
    g = T.backward(d["dy"], d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=c["Q"])
    gs = T.backward(d["dy"][sl], d["x"][sl], d["dt"][sl], d["A"], d["B"][sl], d["C"][sl], d["D"], chunk=c["Q"])
    for k in ("dx", "ddt", "dB", "dC"):
        assert torch.equal(g[k][sl], gs[k]), k


def test_prefill_then_steps_at_full_batch(lib):
    """cfg1 batch: chunk-scan over 896 tokens, then 128 single steps over all 512 x 8 states, against
    the chunk-scan over all 1024 tokens."""
    import trading_bot_0_b200 as T
    c = CFGS["cfg1"]
    d = draw(c)
    y, fin, _ = T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=c["Q"])
    k = 896
    _, s, _ = T.forward(d["x"][:, :k], d["dt"][:, :k], d["A"], d["B"][:, :k], d["C"][:, :k], d["D"], chunk=c["Q"])
    st = T.StreamState(s)
    worst = 0.0
    for t in range(k, c["L"]):
        yt = st.step(d["x"][:, t], d["dt"][:, t], d["A"], d["B"][:, t], d["C"][:, t], d["D"])
        worst = max(worst, (yt.float() - y[:, t].float()).abs().max().item())
    assert worst <= 2e-2
    assert rel(st.state, fin) <= 1e-3


def test_decode_full_rollout_width(lib):
    """8192 streams: one batched step equals the same step done in two halves (stream sharding)."""
    import trading_bot_0_b200 as T
    g = torch.Generator(device=DEV).manual_seed(3)
    S, H, P, N = 8192, 8, 32, 64
    st = 0.1 * torch.randn(S, H, P, N, generator=g, device=DEV)
    x = torch.randn(S, H, P, generator=g, device=DEV).bfloat16()
    dt = F.softplus(torch.randn(S, H, generator=g, device=DEV) - 3).bfloat16()
    A = -torch.exp(torch.rand(H, generator=g, device=DEV) * math.log(16.0))
    Bm = (torch.randn(S, 1, N, generator=g, device=DEV) / 8).bfloat16()
    Cm = (torch.randn(S, 1, N, generator=g, device=DEV) / 8).bfloat16()
    full = st.clone()
    y = T.state_update(full, x, dt, A, Bm, Cm, torch.ones(H, device=DEV))
    halves = [st[:4096].clone(), st[4096:].clone()]
    ys = [T.state_update(halves[i], x[i * 4096:(i + 1) * 4096], dt[i * 4096:(i + 1) * 4096], A,
                         Bm[i * 4096:(i + 1) * 4096], Cm[i * 4096:(i + 1) * 4096], torch.ones(H, device=DEV)) for i in range(2)]
    assert torch.equal(y, torch.cat(ys)) and torch.equal(full, torch.cat(halves))

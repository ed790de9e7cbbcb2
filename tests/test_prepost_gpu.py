"""The operators either side of the scan (causal depthwise conv1d + silu, RMS norm) and the differentiable
composition of the Mamba-2 mixer core, against the fp64 oracle."""
import pytest
import torch

from oracle import ssd_oracle as O
from tests._util import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _autograd_ref(fn, leaves, dout):
    ls = [None if v is None else v.detach().double().requires_grad_(True) for v in leaves]
    out = fn(*ls)
    (out * dout.double()).sum().backward()
    return out.detach(), [None if v is None else v.grad for v in ls]


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("K,activation,use_bias", [(4, True, True), (3, False, False), (2, True, True)])
@pytest.mark.parametrize("Bn,L,Cn", [(3, 200, 384), (2, 130, 200), (2, 64, 24), (1, 7, 8)])
def test_conv1d_forward_backward(lib, dtype, K, activation, use_bias, Bn, L, Cn):
    from trading_bot_0_b200 import prepost as PP
    g = torch.Generator().manual_seed(7)
    td = O.torch_dtype(dtype)
    x = torch.randn(Bn, L, Cn, generator=g).to(td)
    w = torch.randn(Cn, K, generator=g) / K ** 0.5
    b = 0.3 * torch.randn(Cn, generator=g) if use_bias else None
    dout = torch.randn(Bn, L, Cn, generator=g).to(td)
    ref, (dx_r, dw_r, db_r) = _autograd_ref(lambda a, ww, bb: O.causal_conv1d_ref(a, ww, bb, activation), [x, w, b], dout)
    out = PP.conv1d_forward(x.to(DEV), w.to(DEV), None if b is None else b.to(DEV), activation=activation)
    assert_close("out", out, ref, dtype)
    # the gradient arrives as three channel segments when the channel count allows it (multiples of 8)
    c1 = (Cn // 16) * 8
    cuts = [c1, (Cn - c1) // 16 * 8, Cn - c1 - (Cn - c1) // 16 * 8]
    cuts = [c for c in cuts if c > 0]
    segs = [s.contiguous() for s in dout.to(DEV).split(cuts, dim=2)]
    din, dw, db = PP.conv1d_backward(x.to(DEV), w.to(DEV), None if b is None else b.to(DEV), segs, activation=activation)
    assert_close("din", din, dx_r, dtype)
    assert_close("dweight", dw, dw_r, dtype)
    if use_bias:
        assert_close("dbias", db, db_r, dtype)


def test_conv1d_output_views_feed_the_scan(lib):
    """The three channel ranges of the conv output are handed to the scan as strided views (no copies)."""
    import trading_bot_0_b200 as T
    from trading_bot_0_b200 import prepost as PP
    cfg = O.SsdConfig("pp", 2, 256, 8, 32, 64, 1, 128, "bf16", False)
    inp = O.make_inputs(cfg)
    H, P, N, G = 8, 32, 64, 1
    g = torch.Generator().manual_seed(9)
    xBC = torch.randn(2, 256, H * P + 2 * G * N, generator=g).bfloat16()
    w = torch.randn(xBC.shape[2], 4, generator=g) / 2
    u_ref = O.causal_conv1d_ref(xBC, w, None, True)
    u = PP.conv1d_forward(xBC.to(DEV), w.to(DEV), None, activation=True)
    x, Bm, Cm = u.split((H * P, G * N, G * N), dim=2)
    y, fin, _ = T.forward(x.unflatten(2, (H, P)), inp["dt"].to(DEV), inp["A"].to(DEV), Bm.unflatten(2, (G, N)),
                          Cm.unflatten(2, (G, N)), inp["D"].to(DEV), chunk=128, algo="tensor")
    ub = u.cpu()   # the oracle sees the same bf16-rounded conv output
    y_ref, _ = O.ssd_sequential(ub[..., :H * P].reshape(2, 256, H, P), inp["dt"], inp["A"], ub[..., H * P:H * P + N].reshape(2, 256, G, N),
                                ub[..., H * P + N:].reshape(2, 256, G, N), inp["D"])
    assert_close("conv", u, u_ref, "bf16")
    assert_close("y", y, y_ref, "bf16")


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("rows,width,use_weight", [(300, 256, True), (37, 1536, True), (5, 8, False), (64, 2048, False)])
def test_rmsnorm_forward_backward(lib, dtype, rows, width, use_weight):
    from trading_bot_0_b200 import prepost as PP
    g = torch.Generator().manual_seed(3)
    td = O.torch_dtype(dtype)
    x = torch.randn(rows, width, generator=g).to(td)
    w = (1.0 + 0.2 * torch.randn(width, generator=g)) if use_weight else None
    dout = torch.randn(rows, width, generator=g).to(td)
    ref, (dx_r, dw_r) = _autograd_ref(lambda a, ww: O.rmsnorm_ref(a, ww, 1e-5), [x, w], dout)
    out, rstd = PP.rmsnorm_forward(x.to(DEV), None if w is None else w.to(DEV), eps=1e-5)
    assert_close("out", out, ref, dtype)
    din, dw = PP.rmsnorm_backward(x.to(DEV), None if w is None else w.to(DEV), rstd, dout.to(DEV), eps=1e-5)
    assert_close("din", din, dx_r, dtype)
    if use_weight:
        assert_close("dweight", dw, dw_r, dtype)


def test_mamba2_mixer_core_autograd(lib):
    """conv -> scan (softplus(dt + dt_bias), silu(z) gate inside) -> norm, through autograd, against fp64 autograd of the
    oracle composition on the same bf16-rounded inputs (and the same bf16 rounding of the two tensors the operators hand to each
    other in the forward pass)."""
    from trading_bot_0_b200 import prepost as PP
    Bn, L, H, P, N, G = 2, 256, 8, 32, 64, 1
    g = torch.Generator().manual_seed(21)
    hp, gn = H * P, G * N
    xBC = torch.randn(Bn, L, hp + 2 * gn, generator=g).bfloat16()
    dt_raw = (0.5 * torch.randn(Bn, L, H, generator=g)).bfloat16()
    z = torch.randn(Bn, L, H, P, generator=g).bfloat16()
    cw = torch.randn(hp + 2 * gn, 4, generator=g) / 2
    cb = 0.1 * torch.randn(hp + 2 * gn, generator=g)
    dt0 = torch.exp(torch.log(torch.tensor(1e-3)) + torch.rand(H, generator=g) * torch.log(torch.tensor(100.0)))
    dt_bias = dt0 + torch.log(-torch.expm1(-dt0))
    A = -torch.exp(torch.rand(H, generator=g) * torch.log(torch.tensor(16.0)))
    D = torch.ones(H)
    nw = 1.0 + 0.1 * torch.randn(hp, generator=g)
    dout = torch.randn(Bn, L, hp, generator=g).bfloat16()
    kw = dict(nheads=H, headdim=P, dstate=N, ngroups=G)
    leaves = [xBC, dt_raw, z, cw, cb, dt_bias, A, D, nw]
    ref, grads = _autograd_ref(lambda *a: O.mamba2_mixer_core_ref(*a, storage=torch.bfloat16, **kw)[0], leaves, dout)
    dl = [v.to(DEV).requires_grad_(True) for v in leaves]
    out, _ = PP.mamba2_mixer_core(*dl, chunk=128, **kw)
    (out.float() * dout.to(DEV).float()).sum().backward()
    assert_close("out", out, ref, "bf16")
    for name, got, want in zip(("dxBC", "ddt", "dz", "dconv_w", "dconv_b", "ddt_bias", "dA", "dD", "dnorm_w"), dl, grads):
        if name in ("ddt_bias", "dA"):
            # sums over all 512 tokens of per-token terms that mostly cancel (|sum| is ~2 % of the sum of magnitudes): the
            # bf16-mode error of the terms (mean-rel 7e-3, gated above through ddt) adds up like a random walk, so the sum
            # is gated at 6e-2 of its largest entry; the exact-fp32 family gives 2e-3 on the same data
            err = (got.grad.detach().double().cpu() - want).abs().max().item()
            assert err <= 6e-2 * want.abs().max().item(), f"{name}: max-abs {err:.3e}"
        else:
            assert_close(name, got.grad, want, "bf16")


def test_mamba2_mixer_core_autograd_fp32_kernels(lib):
    """The same composition with the exact-fp32 scan kernels: the cancelling sums are tight too."""
    from trading_bot_0_b200 import prepost as PP
    Bn, L, H, P, N, G = 2, 128, 4, 32, 16, 1
    g = torch.Generator().manual_seed(22)
    hp, gn = H * P, G * N
    mk = lambda *s: torch.randn(*s, generator=g)
    xBC, dt_raw, z = mk(Bn, L, hp + 2 * gn).bfloat16(), (0.5 * mk(Bn, L, H)).bfloat16(), mk(Bn, L, H, P).bfloat16()
    cw, cb = mk(hp + 2 * gn, 4) / 2, 0.1 * mk(hp + 2 * gn)
    dt_bias, A, D, nw = mk(H) - 3.0, -torch.exp(torch.rand(H, generator=g) * 2.0), torch.ones(H), 1.0 + 0.1 * mk(hp)
    dout = mk(Bn, L, hp).bfloat16()
    kw = dict(nheads=H, headdim=P, dstate=N, ngroups=G)
    leaves = [xBC, dt_raw, z, cw, cb, dt_bias, A, D, nw]
    ref, grads = _autograd_ref(lambda *a: O.mamba2_mixer_core_ref(*a, storage=torch.bfloat16, **kw)[0], leaves, dout)
    dl = [v.to(DEV).requires_grad_(True) for v in leaves]
    out, _ = PP.mamba2_mixer_core(*dl, chunk=64, algo="fp32_cores", **kw)
    (out.float() * dout.to(DEV).float()).sum().backward()
    assert_close("out", out, ref, "bf16")
    for name, got, want in zip(("dxBC", "ddt", "dz", "dconv_w", "dconv_b", "ddt_bias", "dA", "dD", "dnorm_w"), dl, grads):
        assert_close(name, got.grad.detach(), want, "bf16")

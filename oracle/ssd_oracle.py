"""CPU oracle for the Mamba-2 SSD operator.  TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED: the reference snapshot (CarsonBurke/trading_bot_0) holds no SSD
implementation, golden vector, known-answer test or fixture for this path (only
historical `mamba2_*` timing entries in benchmark_results/bench_20260112_070055.json:6-41),
and the upstream `mamba_ssm` package is neither a pinned dependency (Cargo.lock has no
such crate) nor installed.  This file therefore restates the operator's *definition*:

    a_t = exp(dt[b,t,h] * A[h])
    S_t = a_t * S_{t-1} + dt[b,t,h] * x[b,t,h,:] (outer) B[b,t,g,:]       g = h * G // H
    y_t = S_t @ C[b,t,g,:] + D[h] * x[b,t,h,:]
    y_t <- y_t * silu(z_t)                                  (only when a z gate is given)

Two evaluations are provided, in the style of the reference's "exact slow oracle beside a
fast path" tests (trading_bots/src/torch/pope.rs:112-139 `pope_attention_reference`, the
scalar GAE loop in trading_bots/src/torch/train/gae.rs:155-175):

  * `ssd_sequential`  - the recurrence, one timestep at a time, any float dtype (fp64 is the
                        ground truth); gradients come from torch autograd.
  * `ssd_chunked`     - the four-stage chunked form (cumsum, chunk_state, state_passing,
                        chunk_scan) written with plain torch ops.  Run in fp32 on the host
                        cores it stands in for the reference's "tch on CPU" path (tch is a
                        thin binding over the same libtorch ATen CPU kernels) and is the
                        timed CPU baseline.
  * `ssd_sequential_grads_manual` - a hand-derived reverse recurrence in numpy fp64 that
                        cross-checks autograd (no shared code with it).
  * `state_update`    - one timestep on a caller-owned state, the streamed-rollout step in
                        the slot of `TradingModel::step_on_device`
                        (trading_bots/src/torch/model/stream/live.rs:257-320).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this file.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F

SEED = 20260811  # the reference's default run seed (trading_bots/src/main.rs:120)


@dataclass(frozen=True)
class SsdConfig:
    name: str
    batch: int
    seqlen: int
    nheads: int
    headdim: int
    dstate: int
    ngroups: int
    chunk: int
    dtype: str  # "fp32" | "bf16"
    has_z: bool = False


# The five workload shapes the headline metric is quoted on.
CONFIGS = {
    0: SsdConfig("cfg0_cpu_parity", 4, 256, 4, 32, 16, 1, 64, "fp32"),
    1: SsdConfig("cfg1_policy_train", 512, 1024, 8, 32, 64, 1, 128, "bf16"),
    2: SsdConfig("cfg2_rollout_decode", 8192, 1, 8, 32, 64, 1, 1, "bf16"),
    3: SsdConfig("cfg3_mamba2_130m_layer", 16, 4096, 24, 64, 128, 1, 256, "bf16", True),
    4: SsdConfig("cfg4_long_seq_parallel", 2, 131072, 24, 64, 128, 1, 256, "bf16"),
}


def torch_dtype(name: str) -> torch.dtype:
    return {"fp32": torch.float32, "bf16": torch.bfloat16, "fp64": torch.float64}[name]


def make_inputs(cfg: SsdConfig, seed: int = SEED, *, batch=None, seqlen=None, with_dy=True,
                with_init_state=False):
    """Seeded synthetic inputs with the distributions the workload text gives.

    Draw order is fixed: x; u (per head) -> dt_bias; dt noise; A; B; C; z (if gated); dy;
    init_state.  Everything is drawn in fp32 on CPU, then rounded to the config's storage
    dtype, so the oracle and the CUDA path see the *same rounded values*.
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    Bn = cfg.batch if batch is None else batch
    L = cfg.seqlen if seqlen is None else seqlen
    H, P, N, G = cfg.nheads, cfg.headdim, cfg.dstate, cfg.ngroups
    dt_ = torch_dtype(cfg.dtype)
    x = torch.randn(Bn, L, H, P, generator=g)
    u = torch.rand(H, generator=g)
    dt0 = torch.exp(math.log(1e-3) + u * math.log(100.0))      # softplus(dt_bias), log-uniform [1e-3,1e-1]
    dt_bias = dt0 + torch.log(-torch.expm1(-dt0))               # inverse softplus
    dt = F.softplus(0.5 * torch.randn(Bn, L, H, generator=g) + dt_bias)
    A = -torch.exp(torch.rand(H, generator=g) * math.log(16.0))
    Bm = torch.randn(Bn, L, G, N, generator=g) / math.sqrt(N)
    Cm = torch.randn(Bn, L, G, N, generator=g) / math.sqrt(N)
    D = torch.ones(H)
    out = dict(x=x.to(dt_), dt=dt.to(dt_), A=A, B=Bm.to(dt_), C=Cm.to(dt_), D=D)
    if cfg.has_z:
        out["z"] = torch.randn(Bn, L, H, P, generator=g).to(dt_)
    if with_dy:
        out["dy"] = torch.randn(Bn, L, H, P, generator=g).to(dt_)
    if with_init_state:
        out["init_state"] = 0.1 * torch.randn(Bn, H, P, N, generator=g)
    return out


def dt_preactivation(dt_raw, dt_bias=None, softplus=False, dtype=torch.float64):
    """Step size a Mamba-2 layer feeds the scan: act(dt_raw + dt_bias), act = softplus or identity, and its
    derivative w.r.t. dt_raw (sigmoid for softplus).  The operator definition in the workload text takes the step
    size after this; the fused form takes dt_raw and the per-head bias."""
    v = dt_raw.to(dtype)
    if dt_bias is not None:
        v = v + dt_bias.to(dtype)
    if softplus:
        return F.softplus(v, threshold=20.0), torch.where(v <= 20.0, torch.sigmoid(v), torch.ones_like(v))
    return v, torch.ones_like(v)


def causal_conv1d_ref(inp, weight, bias=None, activation=True, dtype=torch.float64):
    """out[b,t,c] = act(bias[c] + sum_k weight[c,k] * inp[b, t-K+1+k, c]) with zero history; act = silu or identity.
    The depthwise causal convolution a Mamba-2 layer runs over its (x | B | C) channels (differentiable)."""
    x = inp.to(dtype)
    Bn, L, Cn = x.shape
    K = weight.shape[1]
    xp = F.pad(x, (0, 0, K - 1, 0))
    out = torch.zeros(Bn, L, Cn, dtype=dtype)
    for k in range(K):
        out = out + xp[:, k:k + L, :] * weight.to(dtype)[:, k]
    if bias is not None:
        out = out + bias.to(dtype)
    return F.silu(out) if activation else out


def rmsnorm_ref(inp, weight=None, eps=1e-5, dtype=torch.float64):
    """inp * rsqrt(mean(inp^2, last dim) + eps) * weight (differentiable)."""
    x = inp.to(dtype)
    out = x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return out if weight is None else out * weight.to(dtype)


def _round_through(t, storage):
    """Round to the storage dtype of a tensor that crosses an operator boundary, with a straight-through gradient."""
    return t if storage is None else t + (t.detach().to(storage).to(t.dtype) - t.detach())


def mamba2_mixer_core_ref(xBC, dt_raw, z, conv_weight, conv_bias, dt_bias, A, D, norm_weight, *, nheads, headdim, dstate,
                          ngroups, eps=1e-5, init_state=None, dtype=torch.float64, storage=None):
    """conv + silu -> split -> SSD with softplus(dt + dt_bias) and the silu(z) gate -> RMS norm, one timestep at a time
    for the scan (differentiable ground truth of the fused composition).  `storage` (e.g. torch.bfloat16) rounds the two
    tensors that cross operator boundaries in the forward pass (the conv output and the scan output), so that a
    comparison measures the operators and not the quantisation of what they hand to each other."""
    Bn, L, _ = xBC.shape
    hp, gn = nheads * headdim, ngroups * dstate
    u = _round_through(causal_conv1d_ref(xBC, conv_weight, conv_bias, True, dtype), storage)
    x = u[..., :hp].reshape(Bn, L, nheads, headdim)
    Bm = u[..., hp:hp + gn].reshape(Bn, L, ngroups, dstate)
    Cm = u[..., hp + gn:].reshape(Bn, L, ngroups, dstate)
    dt = F.softplus(dt_raw.to(dtype) + dt_bias.to(dtype), threshold=20.0)
    y, S = ssd_sequential(x, dt, A.to(dtype), Bm, Cm, None if D is None else D.to(dtype), None if z is None else z.to(dtype),
                          init_state, dtype=dtype)
    return rmsnorm_ref(_round_through(y, storage).reshape(Bn, L, hp), norm_weight, eps, dtype), S


def make_decode_inputs(cfg: SsdConfig, steps: int, seed: int = SEED, *, streams=None):
    """Per-step fresh draws for the streamed-rollout workload: state ~ N(0, 0.1)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    S = cfg.batch if streams is None else streams
    H, P, N, G = cfg.nheads, cfg.headdim, cfg.dstate, cfg.ngroups
    dt_ = torch_dtype(cfg.dtype)
    state = 0.1 * torch.randn(S, H, P, N, generator=g)
    u = torch.rand(H, generator=g)
    dt0 = torch.exp(math.log(1e-3) + u * math.log(100.0))
    dt_bias = dt0 + torch.log(-torch.expm1(-dt0))
    A = -torch.exp(torch.rand(H, generator=g) * math.log(16.0))
    x = torch.randn(steps, S, H, P, generator=g).to(dt_)
    dt = F.softplus(0.5 * torch.randn(steps, S, H, generator=g) + dt_bias).to(dt_)
    Bm = (torch.randn(steps, S, G, N, generator=g) / math.sqrt(N)).to(dt_)
    Cm = (torch.randn(steps, S, G, N, generator=g) / math.sqrt(N)).to(dt_)
    return dict(state=state, x=x, dt=dt, A=A, B=Bm, C=Cm, D=torch.ones(H))


def _expand_groups(t: torch.Tensor, H: int) -> torch.Tensor:
    """[.., G, N] -> [.., H, N] with head h reading group h*G//H."""
    G = t.shape[-2]
    return t.repeat_interleave(H // G, dim=-2)


def state_update(state, x, dt, A, B, C, D=None, z=None):
    """One timestep.  state [S,H,P,N] (returned, not modified); x [S,H,P]; dt [S,H];
    B, C [S,G,N].  Returns (y [S,H,P], new_state).  Math in state's dtype."""
    f = state.dtype
    H = x.shape[-2]
    x_, dt_ = x.to(f), dt.to(f)
    Bh, Ch = _expand_groups(B.to(f), H), _expand_groups(C.to(f), H)
    a = torch.exp(dt_ * A.to(f))                                      # [S,H]
    new_state = state * a[..., None, None] + (dt_[..., None] * x_)[..., None] * Bh[..., None, :]
    y = torch.einsum("shpn,shn->shp", new_state, Ch)
    if D is not None:
        y = y + D.to(f)[:, None] * x_
    if z is not None:
        y = y * F.silu(z.to(f))
    return y, new_state


def ssd_sequential(x, dt, A, B, C, D=None, z=None, init_state=None, dtype=torch.float64):
    """The recurrence evaluated one timestep at a time in `dtype` (differentiable)."""
    Bn, L, H, P = x.shape
    N = B.shape[-1]
    S = (torch.zeros(Bn, H, P, N, dtype=dtype) if init_state is None else init_state.to(dtype))
    ys = []
    for t in range(L):
        y, S = state_update(S, x[:, t], dt[:, t], A, B[:, t], C[:, t], D,
                            None if z is None else z[:, t])
        ys.append(y)
    return torch.stack(ys, dim=1), S


def ssd_chunked(x, dt, A, B, C, D=None, z=None, init_state=None, chunk=64, dtype=torch.float32):
    """Four-stage chunked evaluation with plain torch ops (differentiable).

    Stage names follow the operator text: cumsum -> chunk_state -> state_passing -> chunk_scan.
    Requires seqlen % chunk == 0.
    """
    f = dtype
    Bn, L, H, P = x.shape
    N = B.shape[-1]
    Q = chunk
    assert L % Q == 0
    nc = L // Q
    xf = x.to(f).view(Bn, nc, Q, H, P)
    dtf = dt.to(f).view(Bn, nc, Q, H)
    Bh = _expand_groups(B.to(f), H).view(Bn, nc, Q, H, N)
    Ch = _expand_groups(C.to(f), H).view(Bn, nc, Q, H, N)
    # cumsum: inclusive within-chunk cumulative sum of dt*A
    cs = torch.cumsum(dtf * A.to(f), dim=2)                                  # [B,nc,Q,H]
    # chunk_state: sum_l exp(cs_end - cs_l) dt_l x_l (outer) B_l
    w = torch.exp(cs[:, :, -1:, :] - cs) * dtf                               # [B,nc,Q,H]
    states = torch.einsum("bclh,bclhp,bclhn->bchpn", w, xf, Bh)
    # state_passing: S_c = exp(cs_end,c) S_{c-1} + states_c ; prev[c] = state entering chunk c
    S = (torch.zeros(Bn, H, P, N, dtype=f) if init_state is None else init_state.to(f))
    prev = []
    for c in range(nc):
        prev.append(S)
        S = torch.exp(cs[:, c, -1, :])[..., None, None] * S + states[:, c]
    prev = torch.stack(prev, dim=1)                                          # [B,nc,H,P,N]
    # chunk_scan
    CB = torch.einsum("bcihn,bcjhn->bchij", Ch, Bh)                          # [B,nc,H,Q,Q]
    cst = cs.permute(0, 1, 3, 2)                                             # [B,nc,H,Q]
    seg = cst[..., :, None] - cst[..., None, :]
    mask = torch.tril(torch.ones(Q, Q, dtype=torch.bool))
    Lm = torch.exp(seg.masked_fill(~mask, float("-inf")))
    M = CB * Lm * dtf.permute(0, 1, 3, 2)[..., None, :]
    y = torch.einsum("bchij,bcjhp->bcihp", M, xf)
    y = y + torch.einsum("bcihn,bchpn->bcihp", Ch, prev) * torch.exp(cs)[..., None]
    if D is not None:
        y = y + D.to(f)[:, None] * xf
    y = y.reshape(Bn, L, H, P)
    if z is not None:
        y = y * F.silu(z.to(f))
    return y, S


def ssd_sequential_grads_manual(x, dt, A, B, C, D, dy, z=None, init_state=None, dfinal=None):
    """Hand-derived reverse recurrence in numpy fp64 (independent of autograd).

    Returns dict(y, final_state, dx, ddt, dA, dB, dC, dD, dz, dinit).
    """
    f = np.float64
    x, dt, A, B, C, D, dy = [t.detach().to(torch.float64).numpy() for t in (x, dt, A, B, C, D, dy)]
    Bn, L, H, P = x.shape
    G, N = B.shape[-2:]
    rep = H // G
    Bh = np.repeat(B, rep, axis=2)
    Ch = np.repeat(C, rep, axis=2)
    zz = None if z is None else z.detach().to(torch.float64).numpy()
    S = np.zeros((Bn, H, P, N), f) if init_state is None else init_state.detach().to(torch.float64).numpy().copy()
    states = np.empty((L + 1, Bn, H, P, N), f)
    states[0] = S
    ypre = np.empty((Bn, L, H, P), f)
    a = np.exp(dt * A)                                                       # [B,L,H]
    for t in range(L):
        S = a[:, t, :, None, None] * S + (dt[:, t, :, None] * x[:, t])[..., None] * Bh[:, t, :, None, :]
        states[t + 1] = S
        ypre[:, t] = np.einsum("bhpn,bhn->bhp", S, Ch[:, t]) + D[:, None] * x[:, t]
    if zz is not None:
        sig = 1.0 / (1.0 + np.exp(-zz))
        silu = zz * sig
        y = ypre * silu
        dz = dy * ypre * (sig * (1.0 + zz * (1.0 - sig)))
        dyp = dy * silu
    else:
        y, dz, dyp = ypre, None, dy
    dS = np.zeros((Bn, H, P, N), f) if dfinal is None else dfinal.detach().to(torch.float64).numpy().copy()
    dx = np.empty_like(x)
    ddt = np.empty_like(dt)
    dBh = np.empty_like(Bh)
    dCh = np.empty_like(Ch)
    dA = np.zeros(H, f)
    dD = np.einsum("blhp,blhp->h", dyp, x)
    for t in range(L - 1, -1, -1):
        St = states[t + 1]
        dCh[:, t] = np.einsum("bhpn,bhp->bhn", St, dyp[:, t])
        dS = dS + dyp[:, t][..., None] * Ch[:, t, :, None, :]                # dL/dS_t
        sb = np.einsum("bhpn,bhn->bhp", dS, Bh[:, t])                         # dS_t . B_t
        dx[:, t] = D[:, None] * dyp[:, t] + dt[:, t, :, None] * sb
        dBh[:, t] = dt[:, t, :, None] * np.einsum("bhpn,bhp->bhn", dS, x[:, t])
        da = np.einsum("bhpn,bhpn->bh", dS, states[t]) * a[:, t]              # dL/d(dt*A)
        ddt[:, t] = np.einsum("bhp,bhp->bh", sb, x[:, t]) + da * A
        dA += np.einsum("bh,bh->h", da, dt[:, t])
        dS = dS * a[:, t, :, None, None]
    dB = dBh.reshape(Bn, L, G, rep, N).sum(3)
    dC = dCh.reshape(Bn, L, G, rep, N).sum(3)
    return dict(y=y, final_state=states[L], dx=dx, ddt=ddt, dA=dA, dB=dB, dC=dC, dD=dD, dz=dz, dinit=dS)


def ssd_grads_autograd(fn, x, dt, A, B, C, D, dy, z=None, init_state=None, dfinal=None,
                       dtype=torch.float64, **kw):
    """Gradients of `fn` (ssd_sequential or ssd_chunked) by autograd, math in `dtype`."""
    leaves = {}
    for k, v in dict(x=x, dt=dt, A=A, B=B, C=C, D=D, z=z, init_state=init_state).items():
        leaves[k] = None if v is None else v.detach().to(dtype).requires_grad_(True)
    y, S = fn(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], leaves["D"],
              leaves["z"], leaves["init_state"], dtype=dtype, **kw)
    loss = (y * dy.to(dtype)).sum()
    if dfinal is not None:
        loss = loss + (S * dfinal.to(dtype)).sum()
    loss.backward()
    out = dict(y=y.detach(), final_state=S.detach())
    for k, v in leaves.items():
        if v is not None:
            out["d" + ("init" if k == "init_state" else k)] = v.grad
    return out

#!/usr/bin/env python
"""Benchmark of the SSD hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg1|cfg2|cfg3|cfg4] [--impl reference]

A step is one pass of the hot path over one batch of seeded synthetic input:
  cfg1 (default, the policy-scale training batch)   forward + backward, metric tokens/s
  cfg3 (Mamba-2-130M layer shapes, gated)           forward + backward, metric tokens/s
  cfg4 (long sequence, sequence-parallel over ranks) forward + backward, metric tokens/s
  cfg2 (streamed rollout, 8192 streams)              one state-update step, metric steps/s
For N > 1 the driver launches one rank per GPU with torch.distributed.run; cfg1/cfg2/cfg3 shard
the batch with no data-path collective (weak scaling: every rank runs the full per-GPU batch),
cfg4 shards the sequence and exchanges slice totals over NCCL.  Rank 0 prints ONE JSON line.

The default line (cfg1) also carries sub-records measured in the same run, so that one line per N holds the whole
picture: `cases` (forward-only, forward+backward, prefill and one decode step, in the result schema of the reference's
benchmark binary, benchmarks/src/results.rs:8-38), `decode` (cfg2, 4096 consecutive steps), `sp_weak` / `sp_strong`
(cfg4 head shapes sharded by sequence over the N ranks, L = 16,384 per rank / L = 131,072 in all) and `sp_check` (one
sequence-parallel forward+backward compared, on rank 0, with the unsplit run of the same inputs on one GPU).

`--impl reference` times the CPU restatement of the same path (plain torch ops on the host
cores, standing in for the reference's tch-on-CPU path, which has no SSD code of its own) on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 20260811
CFGS = {  # B, L, H, P, N, G, Q, has_z
    "cfg1": dict(B=512, L=1024, H=8, P=32, N=64, G=1, Q=128, z=False, name="cfg1_policy_train"),
    "cfg3": dict(B=16, L=4096, H=24, P=64, N=128, G=1, Q=256, z=True, name="cfg3_mamba2_130m_layer"),
    "cfg4": dict(B=2, L=131072, H=24, P=64, N=128, G=1, Q=256, z=False, name="cfg4_long_seq_parallel"),
    "cfg2": dict(B=8192, L=1, H=8, P=32, N=64, G=1, Q=1, z=False, name="cfg2_rollout_decode"),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return float(j["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---- algorithmic bytes (per token / per stream-step) -----------------------------------------
def fwd_bytes_per_token(c, e=2):
    hp, gn = c["H"] * c["P"], c["G"] * c["N"]
    return (hp + c["H"] + 2 * gn + (hp if c["z"] else 0)) * e + hp * e


def bwd_bytes_per_token(c, e=2):
    hp, gn = c["H"] * c["P"], c["G"] * c["N"]
    rd = (hp + c["H"] + 2 * gn + (hp if c["z"] else 0)) * e + hp * e
    wr = hp * e + 4 * c["H"] + 2 * gn * e + (hp * e if c["z"] else 0)
    return rd + wr


def decode_bytes_per_stream(c, e=2):
    return 2 * c["H"] * c["P"] * c["N"] * 4 + (2 * c["H"] * c["P"] + c["H"] + 2 * c["G"] * c["N"]) * e


def kernel_bytes_per_token(name, c, e=2):
    """Bytes of the operator's own inputs/outputs a kernel has to touch, per token; for the two
    scan-over-chunks kernels (whose only operands are the fp32 chunk states) the state traffic."""
    hp, gn, H = c["H"] * c["P"], c["G"] * c["N"], c["H"]
    zb = hp * e if c["z"] else 0
    st = 2 * H * c["P"] * c["N"] * 4 / c["Q"]
    table = {
        "cumsum": H * e, "chunk_state": (hp + gn) * e, "cb": 2 * gn * e,
        # fp32 local states in, bf16 chunk-entry states out; the reverse scan also reads the forward's bf16 copy
        "state_passing": 0.75 * st, "dstate_passing": st, "state_total": st / 2, "dstate_total": st / 2,
        "chunk_scan": (2 * hp + gn) * e + zb, "chunk_scan_bwd_epilogue": (2 * hp + gn) * e + 2 * zb,
        "dstates_local": (hp + gn) * e, "dx": (3 * hp + gn) * e, "dw": 2 * hp * e,
        "dC": (2 * gn + hp) * e, "dB": (2 * gn + hp) * e, "ddt": 4 * H, "sdot": st / 2,
        # tensor-core kernels: each reads its operand tiles once and writes its outputs once
        "chunk_state_tc": (hp + gn) * e, "dstates_local_tc": (hp + gn) * e,
        "chunk_state_ps": (hp + gn) * e, "dstates_local_ps": (hp + gn) * e,
        # chunk states fused with the scan over chunks: the operator's inputs on the way in; the states stay on chip
        "chunk_state_scan": (hp + gn) * e, "dstate_scan": (hp + gn) * e,
        "chunk_scan_tc": (2 * hp + 2 * gn) * e + zb, "chunk_scan_bwd_tc": (2 * hp + 2 * gn) * e + 2 * zb,
        "dx_tc": (3 * hp + 2 * gn) * e, "scan_bwd_dx_tc": (3 * hp + 2 * gn) * e, "dBdC_tc": (2 * hp + 4 * gn) * e,
        "chunk_scan_ws": (2 * hp + 2 * gn) * e + zb, "chunk_scan_bwd_ws": (2 * hp + 2 * gn) * e + 2 * zb,
        "dx_ws": (3 * hp + 2 * gn) * e, "scan_bwd_dx_ws": (3 * hp + 2 * gn) * e, "dBdC_ws": (2 * hp + 4 * gn) * e,
    }
    return table.get(name)


TRAFFIC_SOURCE = ("derived, not measured in this run: dram__bytes_read.sum per token of an ncu capture at batch 128 "
                  "(library as of commit 16fc4c5) scaled by the tokens of a launch, plus the kernel's output bytes; the two "
                  "fused state kernels' figures are that capture minus the fp32 chunk-entry states they no longer move")


def kernel_traffic_bytes_per_token(name, c, e=2):
    """DRAM bytes per token a tensor-family kernel moves at full size: the reads are `dram__bytes_read.sum` of an ncu
    capture of the same kernels at batch 128 (they equal operand tiles + bf16 state boxes + decay tables, each once, and
    grow in proportion to the token count); the writes are the kernel's output bytes, because the writes of the small
    capture partly stay in L2.  A table of constants, stale as soon as a kernel changes its reads: the bench line labels
    it with TRAFFIC_SOURCE.  None where nothing was captured for this shape."""
    if (c["H"], c["P"], c["N"], c["G"], c["Q"], bool(c["z"])) != (8, 32, 64, 1, 128, False) or e != 2:
        return None
    hp, gn, H = c["H"] * c["P"], c["G"] * c["N"], c["H"]
    st32 = H * c["P"] * c["N"] * 4 / c["Q"]          # fp32 chunk states, bytes per token, one way
    measured_reads = {"chunk_state_tc": 768.0, "dstates_local_tc": 768.0, "chunk_scan_ws": 1152.6,
                      "scan_bwd_dx_ws": 1920.6, "dBdC_ws": 1923.1,
                      "chunk_state_scan": 704.6, "dstate_scan": 1216.3 - st32 / 2}   # S_end tile: bf16 now, was fp32
    writes = {"chunk_state_tc": st32, "dstates_local_tc": st32, "chunk_scan_ws": hp * e,
              "scan_bwd_dx_ws": hp * e + 3 * 4 * H, "dBdC_ws": 2 * gn * e,
              "chunk_state_scan": st32 / 2, "dstate_scan": st32 / 2 + 4 * 4 * H / c["Q"]}
    if name not in measured_reads:
        return None
    return measured_reads[name] + writes[name]


# ---- synthetic inputs --------------------------------------------------------------------------
def make_inputs(c, device, seed, dtype=torch.bfloat16, batch=None, seqlen=None):
    """The workload's value distributions, drawn with a seeded generator on `device`."""
    g = torch.Generator(device=device).manual_seed(seed)
    B, L, H, P, N, G = batch or c["B"], seqlen or c["L"], c["H"], c["P"], c["N"], c["G"]
    r = lambda *s: torch.randn(*s, generator=g, device=device)
    x = r(B, L, H, P)
    u = torch.rand(H, generator=g, device=device)
    dt0 = torch.exp(math.log(1e-3) + u * math.log(100.0))
    dt_bias = dt0 + torch.log(-torch.expm1(-dt0))
    dt = F.softplus(0.5 * r(B, L, H) + dt_bias)
    A = -torch.exp(torch.rand(H, generator=g, device=device) * math.log(16.0))
    out = dict(x=x.to(dtype), dt=dt.to(dtype), A=A, B=(r(B, L, G, N) / math.sqrt(N)).to(dtype),
               C=(r(B, L, G, N) / math.sqrt(N)).to(dtype), D=torch.ones(H, device=device))
    if c["z"]:
        out["z"] = r(B, L, H, P).to(dtype)
    out["dy"] = r(B, L, H, P).to(dtype)
    return out


# ---- clocks ------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap,clocks.mem,clocks.max.mem")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.path = gpu_index, None, f"/tmp/ssd_bench_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, pw, mem, mem_mx, reasons = [], [], [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in open(self.path):
            p = [t.strip() for t in line.split(",")]
            if len(p) < 8:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2])); pw.append(float(p[3]))
            except ValueError:
                continue
            for n, v in zip(names, p[4:8]):
                if v == "Active":
                    reasons.add(n)
            try:
                mem.append(float(p[8])); mem_mx.append(float(p[9]))
            except (ValueError, IndexError):
                pass
        try:
            os.remove(self.path)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(pw),
                "mem_mhz": statistics.median(mem) if mem else None, "mem_max_mhz": max(mem_mx) if mem_mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---- CPU baseline (the oracle's chunked torch restatement on the host cores) --------------------
def cpu_fwd_bwd(c, sample_batch, threads, iters=2):
    from oracle import ssd_oracle as O
    torch.set_num_threads(threads)
    inp = make_inputs(c, "cpu", SEED, batch=sample_batch, seqlen=min(c["L"], 16384))
    L = inp["x"].shape[1]

    def once():
        leaves = {k: inp[k].float().requires_grad_(True) for k in ("x", "dt", "A", "B", "C", "D") + (("z",) if c["z"] else ())}
        y, _ = O.ssd_chunked(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], leaves["D"],
                             leaves.get("z"), None, chunk=c["Q"], dtype=torch.float32)
        (y * inp["dy"].float()).sum().backward()

    once()
    t0 = time.perf_counter()
    for _ in range(iters):
        once()
    dt = (time.perf_counter() - t0) / iters
    return sample_batch * L / dt, dt, L


def cpu_decode(c, sample_streams, threads, steps=16):
    from oracle import ssd_oracle as O
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(SEED)
    S, H, P, N, G = sample_streams, c["H"], c["P"], c["N"], c["G"]
    state = 0.1 * torch.randn(S, H, P, N, generator=g)
    A = -torch.exp(torch.rand(H, generator=g) * math.log(16.0))
    D = torch.ones(H)
    xs = torch.randn(steps, S, H, P, generator=g).bfloat16()
    dts = F.softplus(0.5 * torch.randn(steps, S, H, generator=g) - 3.0).bfloat16()
    Bs = (torch.randn(steps, S, G, N, generator=g) / math.sqrt(N)).bfloat16()
    Cs = (torch.randn(steps, S, G, N, generator=g) / math.sqrt(N)).bfloat16()
    with torch.no_grad():
        O.state_update(state, xs[0], dts[0], A, Bs[0], Cs[0], D)
        t0 = time.perf_counter()
        for t in range(steps):
            _, state = O.state_update(state, xs[t], dts[t], A, Bs[t], Cs[t], D)
        dt = (time.perf_counter() - t0) / steps
    return dt


def workload_name(c, workload, world):
    """The `config.workload` string: one per workload, the same in both arms."""
    if workload == "cfg2":
        return f"{c['name']}: {c['B']} streams per GPU, H{c['H']} P{c['P']} N{c['N']} G{c['G']}, fp32 state, bf16 step vectors"
    sp = workload == "cfg4"
    return (f"{c['name']}: B{c['B']} L{c['L']} H{c['H']} P{c['P']} N{c['N']} G{c['G']} Q{c['Q']}"
            f"{' z-gated' if c['z'] else ''} fwd+bwd per GPU" + (" (sequence sharded)" if sp else ""))


def run_reference(args, c):
    """The CPU path on all host cores, bounded sample per step; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cores = os.cpu_count() or 1
    decode = args.workload == "cfg2"
    times = []
    if decode:
        sample = 512
        for _ in range(args.warmup + args.steps):
            times.append(cpu_decode(c, sample, cores, steps=4))
        times = times[args.warmup:]
        step_s = statistics.mean(times) * (c["B"] / sample)      # scaled to the full stream count
        value, unit, metric = 1.0 / step_s, "steps/s", "ssd_decode_steps_per_s"
        desc = f"{sample} of {c['B']} streams per step, time scaled by {c['B'] // sample}"
    else:
        sample = 64 if args.workload == "cfg1" else 1
        for _ in range(args.warmup + args.steps):
            tps, dt, L = cpu_fwd_bwd(c, sample, cores, iters=1)
            times.append(dt)
        times = times[args.warmup:]
        tokens = sample * min(c["L"], 16384)
        value, unit, metric = tokens / statistics.mean(times), "tokens/s", "ssd_fwd_bwd_tokens_per_s"
        desc = f"batch {sample} of {c['B']}, seqlen {min(c['L'], 16384)} of {c['L']}, fwd+bwd, fp32 torch ops"
    line = {"impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(times),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(c, args.workload, args.gpus), "sample": desc},
            "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---- GPU arms ------------------------------------------------------------------------------------
def dist_setup(n):
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def max_over_ranks(ms, world, device):
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def timed(fn, steps, world, device):
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    barrier(world)
    return max_over_ranks(e0.elapsed_time(e1), world, device)


def kernel_profile(fn, reps, device):
    from trading_bot_0_b200 import _lib
    agg = {}
    for _ in range(reps):
        fn()   # keeps the device busy while the profiled pass is enqueued: the first bracket then holds no host time
        with _lib.profile(torch.cuda.current_stream(device).cuda_stream) as p:
            fn()
        for name, ms in p.entries:
            a = agg.setdefault(name, [0, 0.0])
            a[0] += 1
            a[1] += ms
    return {k: (v[0] // reps, v[1] / v[0]) for k, v in agg.items()}   # launches per step, avg ms per launch


# ---- sub-records of the default line -------------------------------------------------------------------------------
def time_fn(fn, reps, world, dev, warm=3):
    for _ in range(warm):
        fn()
    return timed(lambda: fn(), reps, world, dev) / reps


def sub_decode(c2, rank, world, local, steps=4096):
    """cfg2: `steps` consecutive single-timestep updates over 8192 streams per GPU, inputs pre-drawn in HBM."""
    import trading_bot_0_b200 as T
    dev = torch.device("cuda", local)
    S, H, P, N, G = c2["B"], c2["H"], c2["P"], c2["N"], c2["G"]
    g = torch.Generator(device=dev).manual_seed(SEED + 100 + rank)
    ring = 64
    state = 0.1 * torch.randn(S, H, P, N, generator=g, device=dev)
    A = -torch.exp(torch.rand(H, generator=g, device=dev) * math.log(16.0))
    D = torch.ones(H, device=dev)
    u = torch.rand(H, generator=g, device=dev)
    dt0 = torch.exp(math.log(1e-3) + u * math.log(100.0))
    dt_bias = dt0 + torch.log(-torch.expm1(-dt0))
    xs = torch.randn(ring, S, H, P, generator=g, device=dev).bfloat16()
    dts = F.softplus(0.5 * torch.randn(ring, S, H, generator=g, device=dev) + dt_bias).bfloat16()
    Bs = (torch.randn(ring, S, G, N, generator=g, device=dev) / math.sqrt(N)).bfloat16()
    Cs = (torch.randn(ring, S, G, N, generator=g, device=dev) / math.sqrt(N)).bfloat16()
    y = torch.empty(S, H, P, dtype=torch.bfloat16, device=dev)
    st = T.StreamState(state)
    k = [0]

    def step():
        i = k[0] % ring
        k[0] += 1
        st.step(xs[i], dts[i], A, Bs[i], Cs[i], D, y=y)

    for _ in range(8):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step = timed(step, steps, world, dev) / steps
    clocks = sampler.stop() if rank == 0 else None
    peak, peak_kind = peaks()
    bytes_step = decode_bytes_per_stream(c2) * S
    ach = bytes_step / (ms_step * 1e-3) / 1e9
    return {"workload": workload_name(c2, "cfg2", world), "steps": steps, "ms_per_step": ms_step,
            "steps_per_s": world * 1e3 / ms_step, "streams_total": S * world, "scaling": "weak",
            "roofline": {"bound": "hbm", "kernel": "state_update", "achieved": ach, "peak": peak, "unit": "GB/s",
                         "frac": ach / peak, "peak_kind": peak_kind, "algorithmic_bytes_per_launch": bytes_step},
            "clocks": clocks}


def sub_cases(c, inp, dec, ms_fwd_bwd, rank, world, local):
    """The four cases of the reference's benchmark binary for a sequence mixer (forward in training, forward+backward,
    prefill, one decode step; names as in benchmark_results/bench_20260112_070055.json), in its result schema
    {name, time_ms, config{batch, seq_len, dtype}} (benchmarks/src/results.rs:8-20) plus tokens_per_s and the fraction of
    the HBM roofline.  time_ms is per GPU; tokens_per_s is the whole job's."""
    import trading_bot_0_b200 as T
    dev = torch.device("cuda", local)
    dims = T.make_dims(inp["x"], inp["dt"], inp["B"], inp["C"], c["Q"], z=inp.get("z"))
    ws = T.alloc_workspace(dims, dev, backward=True)
    y = torch.empty_like(inp["x"])
    fin = torch.empty(c["B"], c["H"], c["P"], c["N"], dtype=torch.float32, device=dev)
    fwd_train = lambda: T.forward(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], inp.get("z"), chunk=c["Q"],
                                  workspace=ws, y=y, return_final_state=False)
    ws_f = T.alloc_workspace(dims, dev, backward=False)      # forward-sized: inference keeps nothing for a backward
    prefill = lambda: T.forward(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], inp.get("z"), chunk=c["Q"],
                                workspace=ws_f, y=y, final_state=fin)
    ms_f = time_fn(fwd_train, 50, world, dev)
    ms_p = time_fn(prefill, 50, world, dev)
    peak, _ = peaks()
    tokens = c["B"] * c["L"]
    cfgd = {"batch": c["B"], "seq_len": c["L"], "dtype": "bf16"}
    fb, bb = fwd_bytes_per_token(c), bwd_bytes_per_token(c)
    fin_b = c["B"] * c["H"] * c["P"] * c["N"] * 4

    def case(name, ms, nbytes, cfg=cfgd, tok=tokens):
        return {"name": name, "time_ms": ms, "config": cfg, "tokens_per_s": world * tok / (ms * 1e-3),
                "roofline_frac": nbytes / (ms * 1e-3) / 1e9 / peak}

    return [case("ssd_forward_train", ms_f, fb * tokens), case("ssd_fwd_bwd_train", ms_fwd_bwd, (fb + bb) * tokens),
            case("ssd_infer_prefill", ms_p, fb * tokens + fin_b),
            case("ssd_infer_step", dec["ms_per_step"], dec["roofline"]["algorithmic_bytes_per_launch"],
                 {"batch": dec["streams_total"] // world, "seq_len": 1, "dtype": "bf16"}, dec["streams_total"] // world)]


class _LocalOnlyOps:
    """The sequence-parallel stages with the collectives taken out (boundary states are zero): what a rank would take if
    the exchange were free.  The difference to the real step is the exposed cost of the exchange."""

    def __init__(self, real):
        self.real = real
        self.forward, self.backward = real.forward, real.backward

    def exchange(self, direction, local_total, boundary, tensors, chunk, algo, workspace, group, overlap=None, **kw):
        if overlap is not None:
            overlap()
        return torch.zeros_like(local_total)

    def allreduce_params(self, dA, dD, group, **kw):
        return dA, dD


def sub_sp(c4, L_global, rank, world, local, reps, label):
    """cfg4 head shapes with the sequence sharded contiguously over the ranks: forward + backward with the cross-rank
    exclusive prefix scan of the boundary states (the library's NCCL exchange).  One rank: the plain unsharded call."""
    import trading_bot_0_b200 as T
    from trading_bot_0_b200 import sp
    dev = torch.device("cuda", local)
    L_loc = L_global // world
    inp = make_inputs(c4, dev, SEED + 7 + rank, seqlen=L_loc)
    tokens = c4["B"] * L_global
    if world == 1:
        dims = T.make_dims(inp["x"], inp["dt"], inp["B"], inp["C"], c4["Q"])
        ws = T.alloc_workspace(dims, dev, backward=True)
        y, out = torch.empty_like(inp["x"]), {}

        def step():
            T.forward(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], None, chunk=c4["Q"], workspace=ws, y=y,
                      return_final_state=False)
            T.backward(inp["dy"], inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], None, chunk=c4["Q"],
                       workspace=ws, fwd_saved=True, out=out)
        ms = time_fn(step, reps, world, dev)
        return {"workload": f"{label}: B{c4['B']} L{L_global} H{c4['H']} P{c4['P']} N{c4['N']} Q{c4['Q']} fwd+bwd, one rank (no exchange)",
                "ms_per_step": ms, "tokens_per_s": tokens / (ms * 1e-3), "exchange_exposed_ms": 0.0, "ms_local_only": ms}
    ops = sp.default_ops()

    def make_step(o):
        def step():
            yy, fin, ctx = sp.sp_forward(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], None, None,
                                         chunk=c4["Q"], ops=o)
            sp.sp_backward(inp["dy"], ctx, ops=o)
        return step
    ms = time_fn(make_step(ops), reps, world, dev)
    ms_local = time_fn(make_step(_LocalOnlyOps(ops)), reps, world, dev)
    return {"workload": f"{label}: B{c4['B']} L{L_global} ({L_loc} per rank) H{c4['H']} P{c4['P']} N{c4['N']} Q{c4['Q']} fwd+bwd, "
                        f"sequence sharded over {world} ranks, NCCL point-to-point exchange of the boundary records + prefix kernel",
            "ms_per_step": ms, "tokens_per_s": tokens / (ms * 1e-3), "ms_local_only": ms_local,
            "exchange_exposed_ms": ms - ms_local}


def sub_sp_check(c4, rank, world, local):
    """One sequence-parallel forward+backward at cfg4 head shapes (B1, L = 256 per rank) against the unsplit run of the
    same inputs on rank 0's GPU (the unsplit tensor-family path is what the GPU tests gate against the CPU oracle)."""
    import torch.distributed as dist
    import trading_bot_0_b200 as T
    from trading_bot_0_b200 import sp
    dev = torch.device("cuda", local)
    cs = dict(c4, B=1)
    L = 256 * world
    full = make_inputs(cs, dev, SEED + 31, seqlen=L)         # same seed on every rank: every rank holds the whole input
    g = torch.Generator(device=dev).manual_seed(SEED + 32)
    init = 0.1 * torch.randn(1, cs["H"], cs["P"], cs["N"], generator=g, device=dev)
    dfin = 0.1 * torch.randn(1, cs["H"], cs["P"], cs["N"], generator=g, device=dev)
    a, b = sp.slice_bounds(L, world, rank, cs["Q"])
    loc = {k: full[k][:, a:b] for k in ("x", "dt", "B", "C", "dy")}
    if world > 1:
        y, fin, ctx = sp.sp_forward(loc["x"], loc["dt"], full["A"], loc["B"], loc["C"], full["D"], None, init, chunk=cs["Q"],
                                    timeout_s=120.0, tag="sp_check")
        gr = sp.sp_backward(loc["dy"], ctx, dfin)
        T.ssd.workspace_status(ctx.workspace)
        parts = {"y": y, "dx": gr["dx"], "ddt": gr["ddt"], "dB": gr["dB"], "dC": gr["dC"]}
        gathered = {}
        for k, v in parts.items():
            bufs = [torch.empty_like(v) for _ in range(world)]
            dist.all_gather(bufs, v.contiguous())
            gathered[k] = torch.cat(bufs, 1)
        last = torch.empty_like(fin)
        dist.broadcast(fin if rank == world - 1 else last, src=world - 1)
        gathered["final_state"] = fin if rank == world - 1 else last
        gathered.update(dA=gr["dA"], dD=gr["dD"], dinit=gr["dinit"])     # dinit is rank 0's; dA/dD already summed
    if rank != 0:
        return None
    y0, fin0, ws0 = T.forward(full["x"], full["dt"], full["A"], full["B"], full["C"], full["D"], None, init, chunk=cs["Q"],
                              for_backward=True)
    g0 = T.backward(full["dy"], full["x"], full["dt"], full["A"], full["B"], full["C"], full["D"], None, init, dfin,
                    chunk=cs["Q"], workspace=ws0, fwd_saved=True, want_dinit=True, check=True)
    ref = dict(y=y0, final_state=fin0, **{k: g0[k] for k in ("dx", "ddt", "dB", "dC", "dA", "dD", "dinit")})
    if world == 1:
        # one rank: the staged entry points with the library's one-rank exchange against the plain call
        own_group = not dist.is_initialized()
        if own_group:
            dist.init_process_group("gloo", store=dist.HashStore(), rank=0, world_size=1)
        y, fin, ctx = sp.sp_forward(full["x"], full["dt"], full["A"], full["B"], full["C"], full["D"], None, init, chunk=cs["Q"])
        gr = sp.sp_backward(full["dy"], ctx, dfin)
        T.ssd.workspace_status(ctx.workspace)
        gathered = dict(y=y, final_state=fin, **{k: gr[k] for k in ("dx", "ddt", "dB", "dC", "dA", "dD", "dinit")})
        torch.cuda.synchronize()
        if own_group:
            dist.destroy_process_group()
    worst_abs, worst_rel, bad = 0.0, 0.0, []
    for k, r in ref.items():
        got, r = gathered[k].double(), r.double()
        ma = float((got - r).abs().max())
        mr = float((got - r).abs().mean() / (r.abs().mean() + 1e-300))
        scale = max(1.0, float(r.abs().max()))
        worst_abs, worst_rel = max(worst_abs, ma / scale), max(worst_rel, mr)
        if not (ma <= 2e-2 * scale and mr <= 1e-2) or not torch.isfinite(got).all():
            bad.append(k)
    return {"world": world, "seqlen": L, "max_abs": worst_abs, "mean_rel": worst_rel, "ok": not bad, "failed": bad,
            "reference": "unsplit run of the same inputs on rank 0 (tensor-core family, gated against the CPU oracle by the GPU tests)",
            "gate": "2e-2 max-abs (scaled by max(1, max|ref|)) and 1e-2 mean-rel on y, final_state and every gradient"}


def sub_records(args, c, inp, rank, world, local, ms_fwd_bwd):
    out = {}
    dec = sub_decode(CFGS["cfg2"], rank, world, local)
    out["decode"] = dec
    out["cases"] = sub_cases(c, inp, dec, ms_fwd_bwd, rank, world, local)
    torch.cuda.empty_cache()
    c4 = CFGS["cfg4"]
    out["sp_weak"] = sub_sp(c4, 16384 * world, rank, world, local, 10, "cfg4 weak scaling")
    torch.cuda.empty_cache()
    out["sp_strong"] = sub_sp(c4, c4["L"], rank, world, local, 5, "cfg4 strong scaling")
    torch.cuda.empty_cache()
    out["sp_check"] = sub_sp_check(c4, rank, world, local)
    return out


def run_train(args, c, rank, world, local):
    import trading_bot_0_b200 as T
    from trading_bot_0_b200 import _lib
    from trading_bot_0_b200.host import HostFwdBwd
    dev = torch.device("cuda", local)
    sp_mode = args.workload == "cfg4"
    L_loc = c["L"] // world if sp_mode else c["L"]
    inp = make_inputs(c, dev, SEED + rank, seqlen=L_loc)
    z = inp.get("z")
    tokens_rank = c["B"] * L_loc
    dims = T.make_dims(inp["x"], inp["dt"], inp["B"], inp["C"], c["Q"], z=z, algo=args.algo)
    ws = T.alloc_workspace(dims, dev, backward=True)
    y = torch.empty_like(inp["x"])
    out = {}

    if sp_mode and world > 1:
        from trading_bot_0_b200 import sp

        def step():
            yy, fin, ctx = sp.sp_forward(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], z, None,
                                         chunk=c["Q"], algo=args.algo)
            sp.sp_backward(inp["dy"], ctx)
    else:
        def step():
            T.forward(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], z, chunk=c["Q"], algo=args.algo,
                      workspace=ws, y=y, return_final_state=False)
            T.backward(inp["dy"], inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], z, chunk=c["Q"],
                       algo=args.algo, workspace=ws, fwd_saved=True, out=out)

    nwarm = args.warmup if args.profile_mode else max(3, args.warmup)
    for _ in range(nwarm):
        step()
    # one timed step = `inner` passes over the batch, so that the default 20 steps keep the GPU busy for about a second
    # (a clock sampler and the power management see a sustained load, not a 26 ms burst)
    inner = 1 if args.profile_mode else max(1, args.inner)
    pass_once = step

    def step():
        for _ in range(inner):
            pass_once()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    n0 = _lib.launch_count()
    ms = timed(step, args.steps, world, dev)
    launches = _lib.launch_count() - n0
    clocks = sampler.stop() if rank == 0 else None
    ms_step = ms / args.steps
    ms_pass = ms_step / inner
    tokens_job = tokens_rank * world
    value = tokens_job / (ms_pass * 1e-3)

    prof = kernel_profile(pass_once, 3, dev) if not (sp_mode and world > 1) and not args.profile_mode else {}
    host_ms = None
    if not args.profile_mode and not (sp_mode and world > 1):
        # host time of one pass (argument checks, tensor-map encoding, launches) with the device idle behind it
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(10):
            pass_once()
        host_ms = (time.perf_counter() - t0) / 10 * 1e3
        torch.cuda.synchronize()

    # end to end through the host-buffer entry point: pinned host tensors in, pinned host tensors out
    e2e = None
    if not sp_mode and not args.no_e2e:
        hb = HostFwdBwd(c["B"], c["L"], c["H"], c["P"], c["N"], c["G"], c["Q"], torch.bfloat16, has_z=c["z"], device=dev,
                        algo=args.algo)
        hin = {k: inp[k].cpu().pin_memory() for k in ("x", "dt", "B", "C", "dy") + (("z",) if c["z"] else ())}
        hout = {"y": torch.empty_like(hin["x"]), "dx": torch.empty_like(hin["x"]),
                "ddt": torch.empty(c["B"], c["L"], c["H"], dtype=torch.float32).pin_memory(),
                "dB": torch.empty_like(hin["B"]), "dC": torch.empty_like(hin["C"]),
                "dA": torch.empty(c["H"]).pin_memory(), "dD": torch.empty(c["H"]).pin_memory()}
        for k in ("y", "dx", "dB", "dC"):
            hout[k] = hout[k].pin_memory()
        if c["z"]:
            hout["dz"] = torch.empty_like(hin["x"]).pin_memory()
        e2e_step = lambda: hb.run(hin, inp["A"], inp["D"], hout)
        e2e_step()
        e2e_steps = args.steps
        ems = timed(e2e_step, e2e_steps, world, dev) / e2e_steps
        h2d, d2h = hb.bytes_per_call()
        e2e = {"value": tokens_job / (ems * 1e-3), "unit": "tokens/s", "ms_per_step": ems,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
               "h2d_GBps_per_rank": h2d / (ems * 1e-3) / 1e9, "d2h_GBps_per_rank": d2h / (ems * 1e-3) / 1e9,
               "note": "one pass per step; bound by the host<->device copies (both directions at once), not by a kernel"}
        del hb, hin, hout

    subs = {}
    if args.workload == "cfg1" and not args.profile_mode and not args.no_sub:
        subs = sub_records(args, c, inp, rank, world, local, ms_pass)
    if rank != 0:
        return
    peak, peak_kind = peaks()
    roof = None
    if prof:
        dom = max(prof.items(), key=lambda kv: kv[1][0] * kv[1][1])
        name, (n_launch, avg_ms) = dom
        bpt = kernel_bytes_per_token(name, c)
        if bpt is not None:
            ach = bpt * tokens_rank / (avg_ms * 1e-3) / 1e9
            tpt = kernel_traffic_bytes_per_token(name, c)
            roof = {"bound": "hbm", "kernel": name, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                    "peak_kind": peak_kind, "traffic": None if tpt is None else tpt * tokens_rank,
                    "traffic_source": None if tpt is None else TRAFFIC_SOURCE, "avg_launch_ms": avg_ms,
                    "algorithmic_bytes_per_launch": bpt * tokens_rank}
    op_bytes = (fwd_bytes_per_token(c) + bwd_bytes_per_token(c)) * tokens_rank
    op_ach = op_bytes / (ms_pass * 1e-3) / 1e9
    cpu = None
    if world == 1 and not args.no_cpu:
        sample = 64 if args.workload == "cfg1" else 1
        cores = os.cpu_count() or 1
        tps, dt_s, Ls = cpu_fwd_bwd(c, sample, cores, iters=2)
        cpu = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"batch {sample} of {c['B']}, seqlen {Ls} of {c['L']}, fwd+bwd, chunked fp32 torch ops, {dt_s:.2f} s/iter"}
    line = {"metric": "ssd_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": nwarm, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if sp_mode and args.strong else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": workload_name(c, args.workload, world),
                       "algo": args.algo, "passes_per_step": inner, "ms_per_pass": ms_pass,
                       "l2": f"inputs+outputs {op_bytes / 1e6:.0f} MB per pass, larger than the 126 MB L2",
                       "parallelism": "sequence-parallel" if sp_mode else f"batch-sharded x{world}, no collective"},
            "roofline": roof,
            "op_roofline": {"bound": "hbm", "achieved": op_ach, "peak": peak, "unit": "GB/s", "frac": op_ach / peak,
                            "peak_kind": peak_kind, "algorithmic_bytes_per_step": op_bytes},
            "kernels": {k: {"launches_per_pass": v[0], "avg_ms": round(v[1], 5)} for k, v in prof.items()},
            "kernels_note": "CUDA events behind every launch of one pass, enqueued behind an unprofiled pass (no host time in "
                            "any interval); a forward interval includes the memset in front of its kernel",
            "host_ms_per_pass": host_ms,
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks}
    line.update(subs)
    print(json.dumps(line), flush=True)
    if subs.get("sp_check") is not None and not subs["sp_check"]["ok"]:
        sys.exit(3)


def run_decode(args, c, rank, world, local):
    import trading_bot_0_b200 as T
    from trading_bot_0_b200 import _lib
    from trading_bot_0_b200.host import HostStep
    dev = torch.device("cuda", local)
    S, H, P, N, G = c["B"], c["H"], c["P"], c["N"], c["G"]
    g = torch.Generator(device=dev).manual_seed(SEED + rank)
    ring = args.ring                                     # distinct pre-drawn steps held in HBM
    state = 0.1 * torch.randn(S, H, P, N, generator=g, device=dev)
    A = -torch.exp(torch.rand(H, generator=g, device=dev) * math.log(16.0))
    D = torch.ones(H, device=dev)
    u = torch.rand(H, generator=g, device=dev)
    dt0 = torch.exp(math.log(1e-3) + u * math.log(100.0))
    dt_bias = dt0 + torch.log(-torch.expm1(-dt0))
    xs = torch.randn(ring, S, H, P, generator=g, device=dev).bfloat16()
    dts = F.softplus(0.5 * torch.randn(ring, S, H, generator=g, device=dev) + dt_bias).bfloat16()
    Bs = (torch.randn(ring, S, G, N, generator=g, device=dev) / math.sqrt(N)).bfloat16()
    Cs = (torch.randn(ring, S, G, N, generator=g, device=dev) / math.sqrt(N)).bfloat16()
    y = torch.empty(S, H, P, dtype=torch.bfloat16, device=dev)
    st = T.StreamState(state)
    k = [0]

    def step():
        i = k[0] % ring
        k[0] += 1
        st.step(xs[i], dts[i], A, Bs[i], Cs[i], D, y=y)

    nwarm = args.warmup if args.profile_mode else max(3, args.warmup)
    for _ in range(nwarm):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    n0 = _lib.launch_count()
    ms = timed(step, args.steps, world, dev)
    launches = _lib.launch_count() - n0
    clocks = sampler.stop() if rank == 0 else None
    ms_step = ms / args.steps
    if args.profile_mode:
        if rank == 0:
            print(json.dumps({"metric": "ssd_decode_steps_per_s", "value": 1e3 / ms_step, "ms_per_step": ms_step,
                              "profile_mode": True, "gpu_launches": int(launches)}), flush=True)
        return
    prof = kernel_profile(step, 20, dev)
    hs = HostStep(state, G)
    hs.load_inputs(xs[0].cpu(), dts[0].cpu(), Bs[0].cpu(), Cs[0].cpu())   # the step's vectors sit in pinned host memory
    e2e_step = lambda: hs.step(A, D)
    e2e_step()
    e2e_step()
    ems = timed(e2e_step, args.steps, world, dev) / args.steps
    if rank != 0:
        return
    peak, peak_kind = peaks()
    name, (n_launch, ev_ms) = max(prof.items(), key=lambda kv: kv[1][0] * kv[1][1])
    bytes_step = decode_bytes_per_stream(c) * S
    # a step is exactly one launch of this kernel, so the timed region (CUDA events around `steps`
    # back-to-back launches) is its average launch duration; the per-launch event pass is kept as a
    # cross-check (it adds an event record between launches)
    avg_ms = ms_step
    ach = bytes_step / (avg_ms * 1e-3) / 1e9
    cpu = None
    if world == 1 and not args.no_cpu:
        cores = os.cpu_count() or 1
        sample = 512
        dt_s = cpu_decode(c, sample, cores, steps=16)
        cpu = {"value": 1.0 / (dt_s * S / sample), "unit": "steps/s", "cores": cores, "kind": "port",
               "sample": f"{sample} of {S} streams, 16 steps, time scaled by {S // sample}"}
    h2d, d2h = hs.bytes_per_call()
    # unit of work = one step of an 8192-stream rollout; N ranks each advance their own 8192 streams
    line = {"metric": "ssd_decode_steps_per_s", "value": world * 1e3 / ms_step, "unit": "steps/s", "n_gpus": world,
            "steps": args.steps, "warmup": nwarm, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(c, args.workload, world),
                       "streams_total": S * world, "l2": f"state {S * H * P * N * 4 / 1e6:.0f} MB per GPU, larger than the 126 MB L2",
                       "inputs": f"{ring} distinct pre-drawn steps cycled", "parallelism": f"stream-sharded x{world}, no collective"},
            "roofline": {"bound": "hbm", "kernel": name, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "peak_kind": peak_kind, "traffic": None, "avg_launch_ms": avg_ms,
                         "per_launch_event_ms": ev_ms, "algorithmic_bytes_per_launch": bytes_step},
            "cpu_baseline": cpu,
            "e2e": {"value": world * 1e3 / ems, "unit": "steps/s", "ms_per_step": ems, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches), "clocks": clocks}
    print(json.dumps(line), flush=True)


def run_mixer_ops(args, c, rank, world, local):
    """The bandwidth-bound operators either side of the scan (conv1d + silu over the x|B|C channels, RMS norm of the gated
    output), forward and backward, at the cfg1 layer shapes.  A step = the four kernels once over the whole batch."""
    import trading_bot_0_b200  # noqa: F401  (fails loudly without the CUDA library)
    from trading_bot_0_b200 import _lib, prepost as PP
    dev = torch.device("cuda", local)
    B, L, H, P, N, G = c["B"], c["L"], c["H"], c["P"], c["N"], c["G"]
    hp, gn = H * P, G * N
    Cn = hp + 2 * gn
    g = torch.Generator(device=dev).manual_seed(SEED + rank)
    r = lambda *s: torch.randn(*s, generator=g, device=dev)
    xBC, dout_c = r(B, L, Cn).bfloat16(), r(B, L, Cn).bfloat16()
    cw, cb = r(Cn, 4) / 2, 0.1 * r(Cn)
    yg, dout_n, nw = r(B, L, hp).bfloat16(), r(B, L, hp).bfloat16(), 1.0 + 0.1 * r(hp)
    segs = [t.contiguous() for t in dout_c.split((hp, gn, gn), dim=2)]
    _, rstd = PP.rmsnorm_forward(yg, nw)
    ops = {"conv1d_fwd": (lambda: PP.conv1d_forward(xBC, cw, cb), 2 * Cn * 2),
           "conv1d_bwd": (lambda: PP.conv1d_backward(xBC, cw, cb, segs), 3 * Cn * 2),
           "rmsnorm_fwd": (lambda: PP.rmsnorm_forward(yg, nw), 2 * hp * 2 + 4),
           "rmsnorm_bwd": (lambda: PP.rmsnorm_backward(yg, nw, rstd, dout_n), 3 * hp * 2 + 4)}
    step = lambda: [f() for f, _ in ops.values()]
    for _ in range(max(3, args.warmup)):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    n0 = _lib.launch_count()
    ms_step = timed(step, args.steps, world, dev) / args.steps
    launches = _lib.launch_count() - n0
    clocks = sampler.stop() if rank == 0 else None
    per = {k: timed(f, args.steps, world, dev) / args.steps for k, (f, _) in ops.items()}
    if rank != 0:
        return
    peak, peak_kind = peaks()
    tokens = B * L
    kern = {k: {"avg_ms": per[k], "algorithmic_bytes_per_token": ops[k][1],
                "achieved_GBps": ops[k][1] * tokens / (per[k] * 1e-3) / 1e9,
                "frac": ops[k][1] * tokens / (per[k] * 1e-3) / 1e9 / peak} for k in ops}
    dom = max(per, key=per.get)
    cpu = None
    if world == 1 and not args.no_cpu:
        import time as _t
        from oracle import ssd_oracle as O
        torch.set_num_threads(os.cpu_count() or 1)
        sb = 16
        hx, hy = xBC[:sb].float().cpu(), yg[:sb].float().cpu()
        hw, hb, hn = cw.cpu(), cb.cpu(), nw.cpu()
        t0 = _t.perf_counter()
        for t_, fn in ((hx, lambda a: O.causal_conv1d_ref(a, hw, hb, True, torch.float32)), (hy, lambda a: O.rmsnorm_ref(a, hn, 1e-5, torch.float32))):
            a = t_.clone().requires_grad_(True)
            fn(a).sum().backward()
        dt_s = _t.perf_counter() - t0
        cpu = {"value": sb * L / dt_s, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
               "sample": f"batch {sb} of {B}, the four operators through torch CPU ops in fp32, {dt_s:.2f} s"}
    line = {"metric": "mixer_pre_post_ops_tokens_per_s", "value": world * tokens / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"mixer_ops at cfg1 shapes: B{B} L{L}, conv1d width 4 + silu over {Cn} channels, RMS norm over {hp} features, forward + backward per GPU",
                       "l2": f"{tokens * 2 * Cn * 2 / 1e6:.0f} MB moved by the smallest kernel, larger than the 126 MB L2",
                       "parallelism": f"batch-sharded x{world}, no collective"},
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": kern[dom]["achieved_GBps"], "peak": peak, "unit": "GB/s",
                         "frac": kern[dom]["frac"], "peak_kind": peak_kind, "traffic": None, "avg_launch_ms": per[dom]},
            "kernels": kern, "cpu_baseline": cpu, "e2e": None, "gpu_launches": int(launches), "clocks": clocks}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg1", choices=sorted(CFGS) + ["mixer_ops"],
                    help="cfg1..cfg4 as in BASELINE.json; mixer_ops: the conv1d / RMS-norm kernels either side of the scan at cfg1 shapes")
    ap.add_argument("--algo", default="auto", choices=["auto", "fp32_cores", "tensor", "tensor_onetile"])
    ap.add_argument("--ring", type=int, default=64, help="cfg2: distinct pre-drawn steps kept in HBM")
    ap.add_argument("--strong", action="store_true", help="cfg4: label the run strong scaling (fixed global L)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--inner", type=int, default=40, help="passes over the batch inside one timed step (cfg1/cfg3/cfg4)")
    ap.add_argument("--no-sub", action="store_true", help="cfg1: skip the cases / decode / sequence-parallel sub-records")
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch / stream count (profiling a small case)")
    ap.add_argument("--seqlen", type=int, default=0, help="override the sequence length (profiling a small case)")
    ap.add_argument("--profile-mode", action="store_true",
                    help="for captures under a profiler: exactly --warmup warm-ups, no per-kernel event pass, no CPU/e2e legs")
    args = ap.parse_args()
    c = dict(CFGS["cfg1" if args.workload == "mixer_ops" else args.workload])
    if args.batch:
        c["B"] = args.batch
    if args.seqlen:
        c["L"] = args.seqlen
    if args.profile_mode:
        args.no_cpu = args.no_e2e = True
    if args.impl == "reference":
        run_reference(args, c)
        return
    rank, world, local = dist_setup(args.gpus)
    try:
        if args.workload == "cfg2":
            run_decode(args, c, rank, world, local)
        elif args.workload == "mixer_ops":
            run_mixer_ops(args, c, rank, world, local)
        else:
            run_train(args, c, rank, world, local)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    # One JSON line on stdout is the contract, and libraries under this process write to file descriptor 1 on their own
    # (NCCL prints its version there when NCCL_DEBUG is set on the box).  So fd 1 is pointed at stderr for the run, and
    # only this file's prints reach the real stdout.
    _real_stdout = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(_real_stdout, "w", buffering=1)
    main()
    sys.stdout.flush()

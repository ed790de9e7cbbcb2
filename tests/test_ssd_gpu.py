"""Parity of the CUDA SSD forward / backward (through the C ABI) against the CPU oracle."""
import dataclasses

import pytest
import torch

from oracle import ssd_oracle as O
from tests._util import assert_close, cfg_like, max_abs, oracle_all, rel_err, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GRADS = ("dx", "ddt", "dA", "dB", "dC", "dD")


def run_case(cfg, *, with_init=False, with_dfinal=False, use_D=True, algo="auto", seed=O.SEED, seqlen=None,
             batch=None, fwd_saved=False):
    import trading_bot_0_b200 as T
    inp = O.make_inputs(cfg, seed, with_init_state=with_init, seqlen=seqlen, batch=batch)
    if not use_D:
        inp["D"] = None
    Bn, Ln = inp["x"].shape[:2]
    dfinal = None
    if with_dfinal:
        g = torch.Generator().manual_seed(seed + 1)
        dfinal = torch.randn(Bn, cfg.nheads, cfg.headdim, cfg.dstate, generator=g)
    ref = oracle_all(inp, dfinal)
    d = to_dev(inp, DEV)
    y, fin, ws = T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d.get("D"), d.get("z"), d.get("init_state"),
                           chunk=cfg.chunk, algo=algo, for_backward=True)
    g = T.backward(d["dy"], d["x"], d["dt"], d["A"], d["B"], d["C"], d.get("D"), d.get("z"), d.get("init_state"),
                   None if dfinal is None else dfinal.to(DEV), chunk=cfg.chunk, algo=algo,
                   workspace=ws if fwd_saved else None, fwd_saved=fwd_saved, want_dinit=True)
    torch.cuda.synchronize()
    mode = cfg.dtype
    assert_close("y", y, ref["y"], mode)
    assert_close("final_state", fin, ref["final_state"], mode)
    for k in GRADS + ("dinit",) + (("dz",) if cfg.has_z else ()):
        if k == "dD" and not use_D:
            continue
        assert_close(k, g[k], ref[k], mode)
    return y, fin, g, ref


@pytest.mark.parametrize("has_z", [False, True])
@pytest.mark.parametrize("with_state", [False, True])
def test_cfg0_fp32_forward_backward(lib, has_z, with_state):
    cfg = cfg_like(0, has_z=has_z)
    run_case(cfg, with_init=with_state, with_dfinal=with_state)


def test_cfg0_fp32_ssm_part_only(lib):
    """With D = 1 the skip term hides the scan (rms ~0.01 vs ~1); D = None exposes it."""
    run_case(cfg_like(0), use_D=False)


@pytest.mark.parametrize("chunk", [16, 64, 128, 256])
def test_fp32_chunk_invariance(lib, chunk):
    run_case(cfg_like(0, chunk=chunk), with_init=True, with_dfinal=True)


@pytest.mark.parametrize("seqlen", [1, 37, 200, 257])
def test_fp32_ragged_tail(lib, seqlen):
    run_case(cfg_like(0, batch=2), seqlen=seqlen, with_init=True, with_dfinal=True)


def test_fp32_groups_and_odd_dims(lib):
    cfg = O.SsdConfig("odd", 2, 96, 6, 24, 40, 3, 32, "fp32", True)
    run_case(cfg, with_init=True, with_dfinal=True)


def test_fp32_large_dims(lib):
    cfg = O.SsdConfig("large", 1, 512, 2, 128, 256, 1, 256, "fp32")
    run_case(cfg, with_dfinal=True)


def test_fp32_fwd_saved_reuse(lib):
    run_case(cfg_like(0, has_z=True), with_init=True, with_dfinal=True, fwd_saved=True)


@pytest.mark.parametrize("base,batch,seqlen", [(1, 3, 512), (3, 1, 512)])
@pytest.mark.parametrize("use_D", [True, False])
def test_bf16_storage_cuda_core_path(lib, base, batch, seqlen, use_D):
    """bf16 storage through the exact-fp32 kernels (shapes of the policy-scale and 130M-layer
    workloads, reduced batch/length so the oracle finishes in seconds)."""
    cfg = cfg_like(base, batch=batch, seqlen=seqlen)
    run_case(cfg, with_init=True, with_dfinal=True, use_D=use_D, algo="fp32_cores")


def test_strided_views_match_contiguous(lib):
    """Narrowed, non-contiguous inputs (batch/sequence strides) give identical results."""
    import trading_bot_0_b200 as T
    cfg = cfg_like(0)
    inp = to_dev(O.make_inputs(cfg), DEV)
    pad = {k: torch.zeros(v.shape[0] + 1, v.shape[1] + 5, *v.shape[2:], dtype=v.dtype, device=DEV)
           for k, v in inp.items() if k in ("x", "dt", "B", "C", "dy")}
    views = {}
    for k, buf in pad.items():
        views[k] = buf[1:, 3:3 + cfg.seqlen]
        views[k].copy_(inp[k])
        assert not views[k].is_contiguous()
    y0, f0, _ = T.forward(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], chunk=cfg.chunk)
    y1, f1, _ = T.forward(views["x"], views["dt"], inp["A"], views["B"], views["C"], inp["D"], chunk=cfg.chunk)
    g0 = T.backward(inp["dy"], inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], chunk=cfg.chunk)
    g1 = T.backward(views["dy"], views["x"], views["dt"], inp["A"], views["B"], views["C"], inp["D"], chunk=cfg.chunk)
    assert torch.equal(y0, y1) and torch.equal(f0, f1)
    for k in GRADS:
        assert torch.equal(g0[k], g1[k]), k


def test_autograd_function_matches_oracle(lib):
    import trading_bot_0_b200 as T
    cfg = cfg_like(0, has_z=True)
    inp = O.make_inputs(cfg, with_init_state=True)
    ref = oracle_all(inp)
    d = to_dev(inp, DEV)
    leaves = {k: d[k].clone().requires_grad_(True) for k in ("x", "dt", "A", "B", "C", "D", "z", "init_state")}
    y, fin = T.ssd_scan(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], leaves["D"], leaves["z"],
                        leaves["init_state"], chunk=cfg.chunk)
    (y * d["dy"]).sum().backward()
    assert_close("y", y.detach(), ref["y"], "fp32")
    for k, r in (("x", "dx"), ("dt", "ddt"), ("A", "dA"), ("B", "dB"), ("C", "dC"), ("D", "dD"), ("z", "dz"),
                 ("init_state", "dinit")):
        assert_close(r, leaves[k].grad, ref[r], "fp32")


def test_cuda_graph_capture_on_side_stream(lib):
    """Forward + backward captured into a CUDA graph on a non-default stream and replayed: the
    contract the reference's PPO update imposes on anything inside its graph body."""
    import trading_bot_0_b200 as T
    cfg = cfg_like(0, has_z=True)
    d = to_dev(O.make_inputs(cfg), DEV)
    dims = T.make_dims(d["x"], d["dt"], d["B"], d["C"], cfg.chunk, z=d["z"])
    ws = T.alloc_workspace(dims, DEV, backward=True)
    y = torch.empty_like(d["x"])
    fin = torch.empty(cfg.batch, cfg.nheads, cfg.headdim, cfg.dstate, device=DEV)
    out = {}

    def body():
        T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], d["z"], chunk=cfg.chunk, workspace=ws, y=y,
                  final_state=fin)
        T.backward(d["dy"], d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], d["z"], chunk=cfg.chunk,
                   workspace=ws, fwd_saved=True, out=out)

    body()
    torch.cuda.synchronize()
    eager = {k: v.clone() for k, v in out.items() if k != "workspace"}
    y_eager = y.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        body()  # warm-up on the side stream
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            body()
    y.zero_()
    for v in out.values():
        v.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, y_eager)
    for k, v in eager.items():
        assert torch.equal(out[k], v), k


@pytest.mark.parametrize("shape", ["cfg0_fp32_gated", "cfg4_heads_bf16", "cfg1_heads_bf16"])
def test_sequence_parallel_split_emulated(lib, shape):
    """The staged entry points + prefix kernel, driven for W slices on one GPU, reproduce the
    unsplit forward and backward (the cross-rank gather is emulated by stacking).  Run for the exact-fp32 family, for the
    head shapes of the long-sequence workload (H24 P64 N128, chunk 256: the staged tensor-core path the sequence-parallel
    ranks take) and for dstate 64; the backward is driven in the split order the overlapped exchange uses
    (LOCAL_STATES|TOTAL, then LOCAL_REST, then FINISH)."""
    import trading_bot_0_b200 as T
    from trading_bot_0_b200 import _lib as L
    from trading_bot_0_b200.sp import CudaOps, slice_bounds
    if shape == "cfg0_fp32_gated":
        cfg, W, mode, dscale = cfg_like(0, has_z=True, seqlen=512), 4, "fp32", 1.0
    elif shape == "cfg4_heads_bf16":
        cfg, W, mode, dscale = O.SsdConfig("sp4", 1, 768, 24, 64, 128, 1, 256, "bf16", False), 3, "bf16", 0.1
    else:
        cfg, W, mode, dscale = O.SsdConfig("sp1", 2, 512, 8, 32, 64, 1, 128, "bf16", False), 2, "bf16", 0.1
    inp = O.make_inputs(cfg, with_init_state=True)
    dfinal = dscale * torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.dstate, generator=torch.Generator().manual_seed(5))
    ref = oracle_all(inp, dfinal)
    d = to_dev(inp, DEV)
    ops = CudaOps()
    sl = [slice_bounds(cfg.seqlen, W, r, cfg.chunk) for r in range(W)]
    keys = ("x", "dt", "B", "C", "dy") + (("z",) if cfg.has_z else ())
    loc = [{k: d[k][:, a:b] for k in keys} for a, b in sl]
    args = lambda r: (loc[r]["x"], loc[r]["dt"], d["A"], loc[r]["B"], loc[r]["C"], d["D"], loc[r].get("z"))
    st = [ops.forward(L.STAGE_LOCAL | L.STAGE_TOTAL, *args(r), None, cfg.chunk, "auto", None, None, None) for r in range(W)]
    gl = torch.stack([ops.total_logdecay(loc[r]["x"], loc[r]["dt"], d["A"], loc[r]["B"], loc[r]["C"], loc[r].get("z"),
                                         cfg.chunk, "auto", st[r][2]) for r in range(W)])
    gs = torch.stack([s[1] for s in st])
    ys, sin = [], []
    for r in range(W):
        sin.append(ops.prefix_state(gs, gl, W, r, +1, d["init_state"]))
        y, fin, _ = ops.forward(L.STAGE_FINISH, *args(r), sin[r], cfg.chunk, "auto", st[r][2], st[r][0], st[r][1].clone())
        ys.append(y)
    assert_close("y", torch.cat(ys, 1), ref["y"], mode)
    assert_close("final_state", fin, ref["final_state"], mode)
    outs = [dict() for _ in range(W)]
    for r in range(W):
        ops.backward(L.STAGE_LOCAL_STATES | L.STAGE_TOTAL, loc[r]["dy"], *args(r), sin[r], None, cfg.chunk, "auto", st[r][2], outs[r])
    gd = torch.stack([o["dinit"].clone() for o in outs])
    dev_dfinal = dfinal.to(DEV)
    for r in range(W):
        dout = ops.prefix_state(gd, gl, W, r, -1, dev_dfinal)
        ops.backward(L.STAGE_LOCAL_REST, loc[r]["dy"], *args(r), sin[r], None, cfg.chunk, "auto", st[r][2], outs[r])
        ops.backward(L.STAGE_FINISH, loc[r]["dy"], *args(r), sin[r], dout, cfg.chunk, "auto", st[r][2], outs[r])
        assert T.ssd.workspace_status(st[r][2]) == 0
    for k in ("dx", "ddt", "dB", "dC") + (("dz",) if cfg.has_z else ()):
        assert_close(k, torch.cat([o[k] for o in outs], 1), ref[k], mode)
    assert_close("dA", sum(o["dA"] for o in outs), ref["dA"], mode)
    assert_close("dD", sum(o["dD"] for o in outs), ref["dD"], mode)
    assert_close("dinit", outs[0]["dinit"], ref["dinit"], mode)


def test_errors_are_reported_not_faulted(lib):
    import trading_bot_0_b200 as T
    from trading_bot_0_b200 import _lib as L
    cfg = cfg_like(0)
    d = to_dev(O.make_inputs(cfg), DEV)
    with pytest.raises(ValueError):
        T.forward(d["x"], d["dt"][:, :-1], d["A"], d["B"], d["C"], d["D"], chunk=cfg.chunk)
    with pytest.raises(ValueError):
        T.forward(d["x"].cpu(), d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=cfg.chunk)
    with pytest.raises(ValueError):
        T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=512)
    with pytest.raises(L.SsdError) as ei:
        T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=cfg.chunk,
                  workspace=torch.empty(1024, dtype=torch.uint8, device=DEV))
    assert ei.value.code == -4 and "workspace too small" in str(ei.value)
    # the context is still usable afterwards
    y, _, _ = T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=cfg.chunk)
    assert torch.isfinite(y).all()


def test_bounded_wait_runs_out_and_the_context_stays_usable(lib):
    """A wait that nothing satisfies gives up after its bound and reports through a status word; the kernel returns
    normally (no trap, no hang) and the next operator call on the same context is correct."""
    import ctypes as C
    import trading_bot_0_b200 as T
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = lib.ssd_selftest_bounded_wait(C.c_void_p(status.data_ptr()), 2_000_000, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 99
    cfg = O.CONFIGS[0]
    inp = O.make_inputs(cfg)
    y_ref, _ = O.ssd_sequential(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"])
    d = to_dev(inp, DEV)
    y, _, _ = T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=cfg.chunk)
    assert_close("y", y, y_ref, "fp32")


def test_timed_out_wait_is_reported_through_the_status_calls(lib):
    """The self-test's timed-out wait, pointed at the status word of a workspace-shaped buffer: ssd_workspace_status maps the
    word to SSD_ERR_TIMEOUT with the wait-site code in the message, the asynchronous copy + ssd_status_check do the same,
    a healthy workspace reads 0, and nothing faults."""
    import ctypes as C
    import trading_bot_0_b200 as T
    from trading_bot_0_b200 import _lib as L
    ws = torch.zeros(256, dtype=torch.uint8, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert T.ssd.workspace_status(ws) == 0
    assert lib.ssd_selftest_bounded_wait(C.c_void_p(ws.data_ptr()), 2_000_000, stream) == 0
    with pytest.raises(L.SsdError) as ei:
        T.ssd.workspace_status(ws)
    assert ei.value.code == -7 and "99" in str(ei.value)
    code = C.c_int32(-1)
    assert lib.ssd_workspace_status(C.c_void_p(ws.data_ptr()), stream, C.byref(code)) == -7 and code.value == 99
    dst = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert lib.ssd_workspace_status_async(C.c_void_p(ws.data_ptr()), C.c_void_p(dst.data_ptr()), stream) == 0
    torch.cuda.synchronize()
    assert lib.ssd_status_check(int(dst.item())) == -7
    assert lib.ssd_status_check(0) == 0
    # the next operator call clears the word of the workspace it runs in and is correct
    cfg = O.CONFIGS[0]
    inp = O.make_inputs(cfg)
    d = to_dev(inp, DEV)
    y, _, w2 = T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=cfg.chunk, check=True)
    y_ref, _ = O.ssd_sequential(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"])
    assert_close("y", y, y_ref, "fp32")


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_backward_twice_on_one_saved_workspace(lib, dtype):
    """retain_graph-style use: two backward calls on the workspace one forward left (fwd_saved = 1) give the same, correct
    gradients; the CUDA-core backward keeps its per-group W sums apart from the forward's C B^T."""
    import trading_bot_0_b200 as T
    cfg = cfg_like(0, has_z=True, dtype=dtype)
    inp = O.make_inputs(cfg, with_init_state=True)
    ref = oracle_all(inp)
    d = to_dev(inp, DEV)
    args = (d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], d["z"], d["init_state"])
    y, fin, ws = T.forward(*args, chunk=cfg.chunk, algo="fp32_cores", for_backward=True)
    outs = [T.backward(d["dy"], *args, chunk=cfg.chunk, algo="fp32_cores", workspace=ws, fwd_saved=True, want_dinit=True)
            for _ in range(2)]
    torch.cuda.synchronize()
    for k in GRADS + ("dz", "dinit"):
        assert_close(k + " (first)", outs[0][k], ref[k], dtype)
        assert torch.equal(outs[0][k], outs[1][k]), f"{k}: the second backward differs from the first"


def test_misaligned_pointer_is_an_error_code_not_a_fault(lib):
    """A y view that starts 8 bytes into an allocation: the tensor-core family refuses it with SSD_ERR_BAD_ALIGNMENT before
    any launch; the CUDA-core family accepts it."""
    import trading_bot_0_b200 as T
    from trading_bot_0_b200 import _lib as L
    cfg = O.SsdConfig("al", 1, 128, 8, 32, 64, 1, 128, "bf16")
    d = to_dev(O.make_inputs(cfg), DEV)
    n = d["x"].numel()
    y_off = torch.empty(n + 8, dtype=torch.bfloat16, device=DEV)[4:4 + n].view_as(d["x"])
    assert y_off.data_ptr() % 16 == 8
    with pytest.raises(L.SsdError) as ei:
        T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=128, algo="tensor", y=y_off)
    assert ei.value.code == -2 and "16-byte" in str(ei.value)
    y_ok, _, _ = T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=128, algo="tensor")
    y2, _, _ = T.forward(d["x"], d["dt"], d["A"], d["B"], d["C"], d["D"], chunk=128, algo="fp32_cores", y=y_off)
    assert (y2.float() - y_ok.float()).abs().max().item() <= 2e-2

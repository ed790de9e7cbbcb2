//! Tensor-in / Tensor-out SSD operator for a tch-rs program: `forward`, `backward`, `state_update`, the status read and the
//! sequence-parallel exchange, over the raw bindings in `ssd-sys`.
//!
//! Shape of the code follows the reference's FFI wrappers: validate every tensor first and return `anyhow::Error`
//! (`validate` in trading_bots/src/torch/fa4.rs:145-191: rank, device, dtype, unit inner stride, matching batch), then call,
//! then read the error slot (`get_and_reset_last_err`, trading_bots/src/torch/cuda/graph.rs:107-118).  Owning handles are
//! RAII types with `Drop` (like `CudaGraph`, trading_bots/src/torch/cuda/graph.rs:100-105).
//!
//! The CUDA stream: tch-rs does not expose the current stream, so the vendored shim needs one more entry point,
//! `at_cuda_current_stream(device_index) -> *mut c_void` (added the way the reference added `at_cuda_graph_*`,
//! vendor/torch-sys-0.25.0/libtch/torch_api.cpp:378-546); it is declared below and must be provided by the host's libtch.
//!
//! UNBUILT: no cargo / rustc in the image this file was written in.
use anyhow::{bail, Result};
use libc::c_void;
use ssd_sys as sys;
use std::ffi::CStr;
use tch::{Device, Kind, Tensor};

extern "C" {
    /// The CUDA stream libtorch currently launches on for `device_index` (a `cudaStream_t`).
    fn at_cuda_current_stream(device_index: i64) -> *mut c_void;
}

#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Algo {
    Auto,
    Fp32Cores,
    Tensor,
    TensorOneTile,
}

impl Algo {
    fn raw(self) -> i32 {
        match self {
            Algo::Auto => sys::SSD_ALGO_AUTO,
            Algo::Fp32Cores => sys::SSD_ALGO_FP32_CORES,
            Algo::Tensor => sys::SSD_ALGO_TENSOR,
            Algo::TensorOneTile => sys::SSD_ALGO_TENSOR_ONETILE,
        }
    }
}

fn last_error() -> String {
    unsafe { CStr::from_ptr(sys::ssd_last_error()).to_string_lossy().into_owned() }
}

fn check(rc: i32, what: &str) -> Result<()> {
    if rc != sys::SSD_OK {
        bail!("{what}: ssd_b200 error {rc}: {}", last_error());
    }
    Ok(())
}

fn cuda_index(t: &Tensor) -> Result<i64> {
    match t.device() {
        Device::Cuda(i) => Ok(i as i64),
        d => bail!("SSD tensors must be CUDA (there is no CPU path), got {d:?}"),
    }
}

fn dtype_of(t: &Tensor) -> Result<i32> {
    match t.kind() {
        Kind::Float => Ok(sys::SSD_F32),
        Kind::BFloat16 => Ok(sys::SSD_BF16),
        k => bail!("SSD storage dtype must be fp32 or bf16, got {k:?}"),
    }
}

fn ptr(t: &Tensor) -> *mut c_void {
    t.data_ptr()
}

fn opt_ptr(t: Option<&Tensor>) -> *mut c_void {
    t.map(|t| t.data_ptr()).unwrap_or(std::ptr::null_mut())
}

/// A sequence operand [batch, seqlen, ..inner..]: dense inner dims, free batch / sequence strides.
fn check_seq(name: &str, t: &Tensor, shape: &[i64], kind: Kind, device: Device) -> Result<()> {
    if t.size() != shape {
        bail!("SSD {name} must have shape {shape:?}, got {:?}", t.size());
    }
    if t.kind() != kind {
        bail!("SSD {name} must be {kind:?}, got {:?}", t.kind());
    }
    if t.device() != device {
        bail!("SSD {name} must be on {device:?}, got {:?}", t.device());
    }
    let st = t.stride();
    let n = shape.len();
    if st[n - 1] != 1 || (n == 4 && st[2] != shape[3]) {
        bail!("SSD {name}: the inner dimensions must be dense (strides {st:?})");
    }
    Ok(())
}

fn check_f32(name: &str, t: &Tensor, shape: &[i64], device: Device) -> Result<()> {
    if t.size() != shape || t.kind() != Kind::Float || t.device() != device || !t.is_contiguous() {
        bail!("SSD {name} must be a contiguous fp32 tensor of shape {shape:?} on {device:?}");
    }
    Ok(())
}

/// Validate the sequence operands and fill the geometry (the checks of `fa4.rs::validate`, for this operator).
pub fn make_dims(x: &Tensor, dt: &Tensor, b: &Tensor, c: &Tensor, z: Option<&Tensor>, y: Option<&Tensor>, chunk: i64, algo: Algo,
                 dt_softplus: bool) -> Result<sys::SsdDims> {
    if x.dim() != 4 {
        bail!("SSD x must be rank-4 [batch, seqlen, nheads, headdim], got {:?}", x.size());
    }
    if b.dim() != 4 {
        bail!("SSD B must be rank-4 [batch, seqlen, ngroups, dstate], got {:?}", b.size());
    }
    let dev = x.device();
    let index = cuda_index(x)?;
    let kind = x.kind();
    let dtype = dtype_of(x)?;
    let (bn, ln, h, p) = (x.size()[0], x.size()[1], x.size()[2], x.size()[3]);
    let (g, n) = (b.size()[2], b.size()[3]);
    check_seq("x", x, &[bn, ln, h, p], kind, dev)?;
    check_seq("dt", dt, &[bn, ln, h], kind, dev)?;
    check_seq("B", b, &[bn, ln, g, n], kind, dev)?;
    check_seq("C", c, &[bn, ln, g, n], kind, dev)?;
    if h % g != 0 {
        bail!("SSD nheads ({h}) must be a multiple of ngroups ({g})");
    }
    if !(1..=256).contains(&chunk) {
        bail!("SSD chunk must be in [1, 256], got {chunk}");
    }
    let mut d = sys::SsdDims {
        batch: bn as i32, seqlen: ln as i32, nheads: h as i32, headdim: p as i32, dstate: n as i32, ngroups: g as i32,
        chunk: chunk as i32, dtype, algo: algo.raw(), device: index as i32, has_z: z.is_some() as i32,
        dt_softplus: dt_softplus as i32, ..Default::default()
    };
    d.x_stride_b = x.stride()[0]; d.x_stride_l = x.stride()[1];
    d.dt_stride_b = dt.stride()[0]; d.dt_stride_l = dt.stride()[1];
    d.b_stride_b = b.stride()[0]; d.b_stride_l = b.stride()[1];
    d.c_stride_b = c.stride()[0]; d.c_stride_l = c.stride()[1];
    if let Some(z) = z {
        check_seq("z", z, &[bn, ln, h, p], kind, dev)?;
        d.z_stride_b = z.stride()[0]; d.z_stride_l = z.stride()[1];
    }
    if let Some(y) = y {
        check_seq("y/dy", y, &[bn, ln, h, p], kind, dev)?;
        d.y_stride_b = y.stride()[0]; d.y_stride_l = y.stride()[1];
    }
    Ok(d)
}

/// Caller-owned scratch of the forward / backward pass (a uint8 tensor from the torch allocator; the library never allocates).
pub struct Workspace {
    pub buf: Tensor,
}

impl Workspace {
    pub fn new(dims: &sys::SsdDims, device: Device, backward: bool) -> Result<Self> {
        let n = unsafe { sys::ssd_workspace_bytes(dims, if backward { sys::SSD_PASS_BWD } else { sys::SSD_PASS_FWD }) };
        if n == 0 {
            bail!("ssd_workspace_bytes: {}", last_error());
        }
        Ok(Self { buf: Tensor::empty([n as i64], (Kind::Uint8, device)) })
    }
    pub fn bytes(&self) -> usize {
        self.buf.size()[0] as usize
    }
    /// Waits for the current stream, then maps the status word to Ok / Err (a bounded wait inside a kernel ran out).
    pub fn status(&self) -> Result<()> {
        let stream = unsafe { at_cuda_current_stream(cuda_index(&self.buf)?) };
        let mut code = 0i32;
        check(unsafe { sys::ssd_workspace_status(self.buf.data_ptr(), stream, &mut code) }, "ssd_workspace_status")
    }
}

pub struct ForwardOut {
    pub y: Tensor,
    pub final_state: Tensor,
    pub workspace: Workspace,
}

/// y, final_state = SSD(x, dt, A, B, C, D, z, init_state).  The workspace comes back so that `backward` can reuse it.
#[allow(clippy::too_many_arguments)]
pub fn forward(x: &Tensor, dt: &Tensor, a: &Tensor, b: &Tensor, c: &Tensor, d: Option<&Tensor>, z: Option<&Tensor>,
               init_state: Option<&Tensor>, dt_bias: Option<&Tensor>, dt_softplus: bool, chunk: i64, algo: Algo) -> Result<ForwardOut> {
    let y = Tensor::empty_like(x).contiguous();
    let dims = make_dims(x, dt, b, c, z, Some(&y), chunk, algo, dt_softplus)?;
    let dev = x.device();
    let (bn, h, p, n) = (dims.batch as i64, dims.nheads as i64, dims.headdim as i64, dims.dstate as i64);
    check_f32("A", a, &[h], dev)?;
    if let Some(d) = d { check_f32("D", d, &[h], dev)?; }
    if let Some(s) = init_state { check_f32("init_state", s, &[bn, h, p, n], dev)?; }
    if let Some(t) = dt_bias { check_f32("dt_bias", t, &[h], dev)?; }
    let final_state = Tensor::empty([bn, h, p, n], (Kind::Float, dev));
    let ws = Workspace::new(&dims, dev, true)?;
    let ptrs = sys::SsdFwdPtrs {
        x: ptr(x), dt: ptr(dt), A: ptr(a) as *const f32, Bm: ptr(b), Cm: ptr(c), D: opt_ptr(d) as *const f32, z: opt_ptr(z),
        init_state: opt_ptr(init_state) as *const f32, y: ptr(&y), final_state: ptr(&final_state) as *mut f32,
        dt_bias: opt_ptr(dt_bias) as *const f32,
    };
    let stream = unsafe { at_cuda_current_stream(dims.device as i64) };
    check(unsafe { sys::ssd_forward(&dims, &ptrs, ws.buf.data_ptr(), ws.bytes(), stream) }, "ssd_forward")?;
    Ok(ForwardOut { y, final_state, workspace: ws })
}

pub struct Grads {
    pub dx: Tensor,
    pub ddt: Tensor,
    pub da: Tensor,
    pub db: Tensor,
    pub dc: Tensor,
    pub dd: Option<Tensor>,
    pub dz: Option<Tensor>,
    pub dinit_state: Option<Tensor>,
    pub ddt_bias: Option<Tensor>,
}

/// Gradients of `forward`; `workspace` is the one the forward returned (its cumsums and chunk states are reused).
#[allow(clippy::too_many_arguments)]
pub fn backward(dy: &Tensor, x: &Tensor, dt: &Tensor, a: &Tensor, b: &Tensor, c: &Tensor, d: Option<&Tensor>, z: Option<&Tensor>,
                init_state: Option<&Tensor>, dfinal_state: Option<&Tensor>, dt_bias: Option<&Tensor>, dt_softplus: bool,
                chunk: i64, algo: Algo, workspace: &Workspace) -> Result<Grads> {
    let dims = make_dims(x, dt, b, c, z, Some(dy), chunk, algo, dt_softplus)?;
    let dev = x.device();
    let (bn, ln, h, p, n, g) = (dims.batch as i64, dims.seqlen as i64, dims.nheads as i64, dims.headdim as i64, dims.dstate as i64,
                                dims.ngroups as i64);
    check_f32("A", a, &[h], dev)?;
    if let Some(s) = dfinal_state { check_f32("dfinal_state", s, &[bn, h, p, n], dev)?; }
    let opt = (x.kind(), dev);
    let f32o = (Kind::Float, dev);
    let grads = Grads {
        dx: Tensor::empty([bn, ln, h, p], opt), ddt: Tensor::empty([bn, ln, h], f32o), da: Tensor::empty([h], f32o),
        db: Tensor::empty([bn, ln, g, n], opt), dc: Tensor::empty([bn, ln, g, n], opt),
        dd: d.map(|_| Tensor::empty([h], f32o)), dz: z.map(|_| Tensor::empty([bn, ln, h, p], opt)),
        dinit_state: init_state.map(|_| Tensor::empty([bn, h, p, n], f32o)), ddt_bias: dt_bias.map(|_| Tensor::empty([h], f32o)),
    };
    let ptrs = sys::SsdBwdPtrs {
        x: ptr(x), dt: ptr(dt), A: ptr(a) as *const f32, Bm: ptr(b), Cm: ptr(c), D: opt_ptr(d) as *const f32, z: opt_ptr(z),
        init_state: opt_ptr(init_state) as *const f32, dy: ptr(dy), dfinal_state: opt_ptr(dfinal_state) as *const f32,
        dx: ptr(&grads.dx), ddt: ptr(&grads.ddt) as *mut f32, dA: ptr(&grads.da) as *mut f32, dB: ptr(&grads.db), dC: ptr(&grads.dc),
        dD: opt_ptr(grads.dd.as_ref()) as *mut f32, dz: opt_ptr(grads.dz.as_ref()), dinit_state: opt_ptr(grads.dinit_state.as_ref()) as *mut f32,
        fwd_saved: 1, dt_bias: opt_ptr(dt_bias) as *const f32, ddt_bias: opt_ptr(grads.ddt_bias.as_ref()) as *mut f32,
    };
    let stream = unsafe { at_cuda_current_stream(dims.device as i64) };
    check(unsafe { sys::ssd_backward(&dims, &ptrs, workspace.buf.data_ptr(), workspace.bytes(), stream) }, "ssd_backward")?;
    Ok(grads)
}

/// One timestep over all streams, in place on `state` [streams, nheads, headdim, dstate] fp32: the slot of
/// `TradingModel::step_on_device` (trading_bots/src/torch/model/stream/live.rs:257-320).  Returns y [streams, nheads, headdim].
#[allow(clippy::too_many_arguments)]
pub fn state_update(state: &mut Tensor, x: &Tensor, dt: &Tensor, a: &Tensor, b: &Tensor, c: &Tensor, d: Option<&Tensor>,
                    z: Option<&Tensor>, dt_bias: Option<&Tensor>, dt_softplus: bool) -> Result<Tensor> {
    if state.dim() != 4 || state.kind() != Kind::Float || !state.is_contiguous() {
        bail!("SSD state must be a contiguous fp32 [streams, nheads, headdim, dstate] tensor, got {:?} {:?}", state.size(), state.kind());
    }
    let dev = state.device();
    let index = cuda_index(state)?;
    let (s, h, p, n) = (state.size()[0], state.size()[1], state.size()[2], state.size()[3]);
    if b.dim() != 3 || b.size()[0] != s || b.size()[2] != n {
        bail!("SSD step B must be [streams, ngroups, dstate], got {:?}", b.size());
    }
    let g = b.size()[1];
    let kind = x.kind();
    for (name, t, shape) in [("x", x, vec![s, h, p]), ("dt", dt, vec![s, h]), ("B", b, vec![s, g, n]), ("C", c, vec![s, g, n])] {
        if t.size() != shape || t.kind() != kind || t.device() != dev || *t.stride().last().unwrap() != 1 {
            bail!("SSD step {name} must be {shape:?} {kind:?} on {dev:?} with a dense inner dimension");
        }
    }
    check_f32("A", a, &[h], dev)?;
    let y = Tensor::empty([s, h, p], (kind, dev));
    let dims = sys::SsdStepDims {
        streams: s as i32, nheads: h as i32, headdim: p as i32, dstate: n as i32, ngroups: g as i32, dtype: dtype_of(x)?,
        device: index as i32, dt_softplus: dt_softplus as i32, x_stride_s: x.stride()[0], dt_stride_s: dt.stride()[0],
        b_stride_s: b.stride()[0], c_stride_s: c.stride()[0], z_stride_s: z.map(|z| z.stride()[0]).unwrap_or(0), y_stride_s: y.stride()[0],
    };
    let ptrs = sys::SsdStepPtrs {
        state: ptr(state) as *mut f32, x: ptr(x), dt: ptr(dt), A: ptr(a) as *const f32, Bm: ptr(b), Cm: ptr(c),
        D: opt_ptr(d) as *const f32, z: opt_ptr(z), y: ptr(&y), dt_bias: opt_ptr(dt_bias) as *const f32,
    };
    let stream = unsafe { at_cuda_current_stream(index) };
    check(unsafe { sys::ssd_state_update(&dims, &ptrs, stream) }, "ssd_state_update")?;
    Ok(y)
}

/// Zero the state rows of finished environments without a host sync (indexed reset, trading_bots/src/torch/model/stream/live.rs:114-158).
pub fn reset_streams(state: &mut Tensor, stream_idx: &Tensor) -> Result<()> {
    if stream_idx.kind() != Kind::Int64 || stream_idx.device() != state.device() {
        bail!("stream_idx must be an int64 tensor on the state's device");
    }
    let streams = state.size()[0];
    let row = state.numel() as i64 / streams;
    let stream = unsafe { at_cuda_current_stream(cuda_index(state)?) };
    check(unsafe { sys::ssd_state_reset_rows(ptr(state) as *mut f32, row, ptr(stream_idx) as *const i64, stream_idx.numel() as i64, streams, stream) },
          "ssd_state_reset_rows")
}

/// Sequence-parallel communicator (NCCL inside the library): new / free pair behind `Drop`.
pub struct SpComm {
    raw: *mut sys::SsdSpComm,
}

unsafe impl Send for SpComm {}

impl SpComm {
    /// Rank 0 draws the id; the host program carries the 128 bytes to the other ranks by its own means.
    pub fn unique_id() -> Result<[u8; sys::SSD_SP_UNIQUE_ID_BYTES]> {
        let mut id = [0u8; sys::SSD_SP_UNIQUE_ID_BYTES];
        check(unsafe { sys::ssd_sp_unique_id(id.as_mut_ptr() as *mut c_void) }, "ssd_sp_unique_id")?;
        Ok(id)
    }
    /// Collective over all ranks, on the current CUDA device.
    pub fn new(id: &[u8; sys::SSD_SP_UNIQUE_ID_BYTES], world: i32, rank: i32) -> Result<Self> {
        let raw = unsafe { sys::ssd_sp_comm_new(id.as_ptr() as *const c_void, world, rank) };
        if raw.is_null() {
            bail!("ssd_sp_comm_new: {}", last_error());
        }
        Ok(Self { raw })
    }
    pub fn world(&self) -> i32 { unsafe { sys::ssd_sp_comm_world(self.raw) } }
    pub fn rank(&self) -> i32 { unsafe { sys::ssd_sp_comm_rank(self.raw) } }
    /// After the LOCAL|TOTAL stages: the state entering this rank's slice (forward, `direction` +1) or the state gradient
    /// leaving it (backward, -1).  `timeout_ms` 0 = enqueue only; > 0 = checked mode (see the header).
    pub fn exchange(&self, dims: &sys::SsdDims, workspace: &Workspace, direction: i32, local_total: &Tensor, boundary: Option<&Tensor>,
                    timeout_ms: i32) -> Result<Tensor> {
        let dev = local_total.device();
        let nbytes = unsafe { sys::ssd_sp_exchange_bytes(dims, self.world()) };
        if nbytes == 0 {
            bail!("ssd_sp_exchange_bytes: {}", last_error());
        }
        let exch = Tensor::empty([nbytes as i64], (Kind::Uint8, dev));
        let out = Tensor::empty_like(local_total);
        let stream = unsafe { at_cuda_current_stream(dims.device as i64) };
        let f = if direction > 0 { sys::ssd_sp_exchange_fwd } else { sys::ssd_sp_exchange_bwd };
        check(unsafe {
            f(dims, workspace.buf.data_ptr(), workspace.bytes(), self.raw, ptr(local_total) as *const f32, opt_ptr(boundary) as *const f32,
              ptr(&out) as *mut f32, exch.data_ptr(), nbytes, stream, timeout_ms)
        }, "ssd_sp_exchange")?;
        Ok(out)
    }
    /// dA / dD summed over the ranks, in place (the parameters are replicated).
    pub fn allreduce_params(&self, da: &mut Tensor, dd: Option<&mut Tensor>, timeout_ms: i32) -> Result<()> {
        let stream = unsafe { at_cuda_current_stream(cuda_index(da)?) };
        let h = da.numel() as i32;
        let ddp = dd.map(|t| t.data_ptr()).unwrap_or(std::ptr::null_mut());
        check(unsafe { sys::ssd_sp_allreduce_params(self.raw, da.data_ptr() as *mut f32, ddp as *mut f32, h, stream, timeout_ms) },
              "ssd_sp_allreduce_params")
    }
    /// After a timeout the communicator is in an unknown state: abort it and make a new one.
    pub fn abort(&mut self) -> Result<()> {
        check(unsafe { sys::ssd_sp_comm_abort(self.raw) }, "ssd_sp_comm_abort")
    }
}

impl Drop for SpComm {
    fn drop(&mut self) {
        unsafe { sys::ssd_sp_comm_free(self.raw) }
    }
}

#[cfg(test)]
mod tests {
    use super::*;

    #[test]
    fn rejects_cpu_tensors_before_any_ffi_call() {
        let x = Tensor::zeros([1, 8, 2, 4], (Kind::Float, Device::Cpu));
        let dt = Tensor::zeros([1, 8, 2], (Kind::Float, Device::Cpu));
        let b = Tensor::zeros([1, 8, 1, 4], (Kind::Float, Device::Cpu));
        assert!(make_dims(&x, &dt, &b, &b, None, None, 8, Algo::Auto, false).is_err());
    }
}

//! Raw bindings to `libssd_b200` (include/ssd_b200.h), one declaration per header entry, in header order.
//!
//! Written to the conventions of the reference's vendored `torch-sys` extern block
//! (vendor/torch-sys-0.25.0/src/lib.rs:34-104: plain `extern "C"`, opaque `#[repr(C)]` handle types with a private
//! zero-sized field, `c_int`-style scalars).  Every pointer is a raw CUDA device pointer as `at_data_ptr` returns it for a
//! tch tensor, except where a comment says host.
//!
//! UNBUILT: the image these files were written in has no cargo / rustc.  A test of the repository
//! (tests/test_rust_layout_cpu.py) parses this file and the header and asserts that every struct has the same fields in
//! the same order with the same widths and that every function has the same name, argument list and return type.
#![allow(non_camel_case_types, non_snake_case)]

use libc::{c_char, c_void, size_t};

// ---- enums (values as in the header) ---------------------------------------------------------------------------
pub const SSD_OK: i32 = 0;
pub const SSD_ERR_BAD_SHAPE: i32 = -1;
pub const SSD_ERR_BAD_ALIGNMENT: i32 = -2;
pub const SSD_ERR_UNSUPPORTED: i32 = -3;
pub const SSD_ERR_WORKSPACE_TOO_SMALL: i32 = -4;
pub const SSD_ERR_CUDA: i32 = -5;
pub const SSD_ERR_NULL_POINTER: i32 = -6;
pub const SSD_ERR_TIMEOUT: i32 = -7;

pub const SSD_F32: i32 = 0;
pub const SSD_BF16: i32 = 1;

pub const SSD_PASS_FWD: i32 = 0;
pub const SSD_PASS_BWD: i32 = 1;

pub const SSD_ALGO_AUTO: i32 = 0;
pub const SSD_ALGO_FP32_CORES: i32 = 1;
pub const SSD_ALGO_TENSOR: i32 = 2;
pub const SSD_ALGO_TENSOR_ONETILE: i32 = 3;

pub const SSD_STAGE_LOCAL: i32 = 1;
pub const SSD_STAGE_TOTAL: i32 = 2;
pub const SSD_STAGE_FINISH: i32 = 4;
pub const SSD_STAGE_LOCAL_STATES: i32 = 8;
pub const SSD_STAGE_LOCAL_REST: i32 = 16;

pub const SSD_SP_UNIQUE_ID_BYTES: usize = 128;
pub const SSD_NOALLOC_MAX_BYTES: usize = 32 << 20;

// ---- structs ---------------------------------------------------------------------------------------------------
#[repr(C)]
#[derive(Debug, Clone, Copy, Default)]
pub struct SsdDims {
    pub batch: i32,
    pub seqlen: i32,
    pub nheads: i32,
    pub headdim: i32,
    pub dstate: i32,
    pub ngroups: i32,
    pub chunk: i32,
    pub dtype: i32,
    pub algo: i32,
    pub device: i32,
    pub has_z: i32,
    pub dt_softplus: i32,
    pub x_stride_b: i64,
    pub x_stride_l: i64,
    pub dt_stride_b: i64,
    pub dt_stride_l: i64,
    pub b_stride_b: i64,
    pub b_stride_l: i64,
    pub c_stride_b: i64,
    pub c_stride_l: i64,
    pub z_stride_b: i64,
    pub z_stride_l: i64,
    pub y_stride_b: i64,
    pub y_stride_l: i64,
}

#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct SsdFwdPtrs {
    pub x: *const c_void,
    pub dt: *const c_void,
    pub A: *const f32,
    pub Bm: *const c_void,
    pub Cm: *const c_void,
    pub D: *const f32,
    pub z: *const c_void,
    pub init_state: *const f32,
    pub y: *mut c_void,
    pub final_state: *mut f32,
    pub dt_bias: *const f32,
}

#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct SsdBwdPtrs {
    pub x: *const c_void,
    pub dt: *const c_void,
    pub A: *const f32,
    pub Bm: *const c_void,
    pub Cm: *const c_void,
    pub D: *const f32,
    pub z: *const c_void,
    pub init_state: *const f32,
    pub dy: *const c_void,
    pub dfinal_state: *const f32,
    pub dx: *mut c_void,
    pub ddt: *mut f32,
    pub dA: *mut f32,
    pub dB: *mut c_void,
    pub dC: *mut c_void,
    pub dD: *mut f32,
    pub dz: *mut c_void,
    pub dinit_state: *mut f32,
    pub fwd_saved: i32,
    pub dt_bias: *const f32,
    pub ddt_bias: *mut f32,
}

#[repr(C)]
#[derive(Debug, Clone, Copy, Default)]
pub struct SsdStepDims {
    pub streams: i32,
    pub nheads: i32,
    pub headdim: i32,
    pub dstate: i32,
    pub ngroups: i32,
    pub dtype: i32,
    pub device: i32,
    pub dt_softplus: i32,
    pub x_stride_s: i64,
    pub dt_stride_s: i64,
    pub b_stride_s: i64,
    pub c_stride_s: i64,
    pub z_stride_s: i64,
    pub y_stride_s: i64,
}

#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct SsdStepPtrs {
    pub state: *mut f32,
    pub x: *const c_void,
    pub dt: *const c_void,
    pub A: *const f32,
    pub Bm: *const c_void,
    pub Cm: *const c_void,
    pub D: *const f32,
    pub z: *const c_void,
    pub y: *mut c_void,
    pub dt_bias: *const f32,
}

/// Opaque owning handle of the sequence-parallel communicator (new / free pair, like `C_cuda_graph`).
#[repr(C)]
pub struct SsdSpComm {
    _private: [u8; 0],
}

#[repr(C)]
#[derive(Debug, Clone, Copy, Default)]
pub struct SsdConvDims {
    pub batch: i32,
    pub seqlen: i32,
    pub channels: i32,
    pub width: i32,
    pub dtype: i32,
    pub device: i32,
    pub activation: i32,
    pub reserved: i32,
    pub in_stride_b: i64,
    pub in_stride_l: i64,
    pub out_stride_b: i64,
    pub out_stride_l: i64,
}

#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct SsdConvGrad {
    pub ptr: *const c_void,
    pub channels: i32,
    pub reserved: i32,
    pub stride_b: i64,
    pub stride_l: i64,
}

#[repr(C)]
#[derive(Debug, Clone, Copy, Default)]
pub struct SsdNormDims {
    pub rows: i64,
    pub width: i32,
    pub dtype: i32,
    pub device: i32,
    pub eps: f32,
    pub in_stride_row: i64,
    pub out_stride_row: i64,
}

// ---- functions (header order) ------------------------------------------------------------------------------------
extern "C" {
    pub fn ssd_workspace_bytes(dims: *const SsdDims, pass: i32) -> size_t;
    pub fn ssd_forward(
        dims: *const SsdDims,
        p: *const SsdFwdPtrs,
        workspace: *mut c_void,
        workspace_bytes: size_t,
        cuda_stream: *mut c_void,
    ) -> i32;
    pub fn ssd_backward(
        dims: *const SsdDims,
        p: *const SsdBwdPtrs,
        workspace: *mut c_void,
        workspace_bytes: size_t,
        cuda_stream: *mut c_void,
    ) -> i32;
    pub fn ssd_state_update(dims: *const SsdStepDims, p: *const SsdStepPtrs, cuda_stream: *mut c_void) -> i32;
    pub fn ssd_state_reset_rows(
        state: *mut f32,
        row_elems: i64,
        stream_idx: *const i64,
        count: i64,
        streams: i64,
        cuda_stream: *mut c_void,
    ) -> i32;
    pub fn ssd_forward_staged(
        dims: *const SsdDims,
        p: *const SsdFwdPtrs,
        workspace: *mut c_void,
        workspace_bytes: size_t,
        cuda_stream: *mut c_void,
        stages: i32,
    ) -> i32;
    pub fn ssd_backward_staged(
        dims: *const SsdDims,
        p: *const SsdBwdPtrs,
        workspace: *mut c_void,
        workspace_bytes: size_t,
        cuda_stream: *mut c_void,
        stages: i32,
    ) -> i32;
    pub fn ssd_sp_total_logdecay(
        dims: *const SsdDims,
        workspace: *const c_void,
        workspace_bytes: size_t,
        out: *mut f32,
        cuda_stream: *mut c_void,
    ) -> i32;
    pub fn ssd_sp_prefix_state(
        gathered_states: *const f32,
        gathered_logdecay: *const f32,
        world: i32,
        rank: i32,
        direction: i32,
        batch_heads: i64,
        state_elems: i64,
        boundary: *const f32,
        state_in: *mut f32,
        cuda_stream: *mut c_void,
    ) -> i32;
    /// `id128`: HOST buffer of SSD_SP_UNIQUE_ID_BYTES bytes.
    pub fn ssd_sp_unique_id(id128: *mut c_void) -> i32;
    pub fn ssd_sp_comm_new(id128: *const c_void, world: i32, rank: i32) -> *mut SsdSpComm;
    pub fn ssd_sp_comm_wrap(nccl_comm: *mut c_void) -> *mut SsdSpComm;
    pub fn ssd_sp_comm_world(comm: *const SsdSpComm) -> i32;
    pub fn ssd_sp_comm_rank(comm: *const SsdSpComm) -> i32;
    pub fn ssd_sp_comm_free(comm: *mut SsdSpComm);
    pub fn ssd_sp_comm_abort(comm: *mut SsdSpComm) -> i32;
    pub fn ssd_sp_exchange_bytes(dims: *const SsdDims, world: i32) -> size_t;
    pub fn ssd_sp_exchange_fwd(
        dims: *const SsdDims,
        workspace: *const c_void,
        workspace_bytes: size_t,
        comm: *mut SsdSpComm,
        local_final_state: *const f32,
        init_state: *const f32,
        state_in: *mut f32,
        exchange_buf: *mut c_void,
        exchange_bytes: size_t,
        cuda_stream: *mut c_void,
        timeout_ms: i32,
    ) -> i32;
    pub fn ssd_sp_exchange_bwd(
        dims: *const SsdDims,
        workspace: *const c_void,
        workspace_bytes: size_t,
        comm: *mut SsdSpComm,
        local_dinit_state: *const f32,
        dfinal_state: *const f32,
        dstate_out: *mut f32,
        exchange_buf: *mut c_void,
        exchange_bytes: size_t,
        cuda_stream: *mut c_void,
        timeout_ms: i32,
    ) -> i32;
    pub fn ssd_sp_allreduce_params(
        comm: *mut SsdSpComm,
        dA: *mut f32,
        dD: *mut f32,
        nheads: i32,
        cuda_stream: *mut c_void,
        timeout_ms: i32,
    ) -> i32;
    /// HOST string, valid until the next call on this thread; not to be freed (unlike libtch's `get_and_reset_last_err`).
    pub fn ssd_last_error() -> *const c_char;
    pub fn ssd_forward_noalloc(dims: *const SsdDims, p: *const SsdFwdPtrs, cuda_stream: *mut c_void) -> i32;
    pub fn ssd_noalloc_max_bytes() -> size_t;
    pub fn ssd_conv1d_workspace_bytes(dims: *const SsdConvDims) -> size_t;
    pub fn ssd_conv1d_forward(
        dims: *const SsdConvDims,
        r#in: *const c_void,
        weight: *const f32,
        bias: *const f32,
        out: *mut c_void,
        cuda_stream: *mut c_void,
    ) -> i32;
    pub fn ssd_conv1d_backward(
        dims: *const SsdConvDims,
        r#in: *const c_void,
        weight: *const f32,
        bias: *const f32,
        dout: *const SsdConvGrad,
        ndout: i32,
        din: *mut c_void,
        din_stride_b: i64,
        din_stride_l: i64,
        dweight: *mut f32,
        dbias: *mut f32,
        workspace: *mut c_void,
        workspace_bytes: size_t,
        cuda_stream: *mut c_void,
    ) -> i32;
    pub fn ssd_rmsnorm_workspace_bytes(dims: *const SsdNormDims) -> size_t;
    pub fn ssd_rmsnorm_forward(
        dims: *const SsdNormDims,
        r#in: *const c_void,
        weight: *const f32,
        out: *mut c_void,
        rstd: *mut f32,
        cuda_stream: *mut c_void,
    ) -> i32;
    pub fn ssd_rmsnorm_backward(
        dims: *const SsdNormDims,
        r#in: *const c_void,
        weight: *const f32,
        rstd: *const f32,
        dout: *const c_void,
        dout_stride_row: i64,
        din: *mut c_void,
        din_stride_row: i64,
        dweight: *mut f32,
        workspace: *mut c_void,
        workspace_bytes: size_t,
        cuda_stream: *mut c_void,
    ) -> i32;
    pub fn ssd_selftest_bounded_wait(device_status: *mut i32, max_cycles: i64, cuda_stream: *mut c_void) -> i32;
    /// `code_out`: HOST int32, optional.
    pub fn ssd_workspace_status(workspace: *const c_void, cuda_stream: *mut c_void, code_out: *mut i32) -> i32;
    pub fn ssd_workspace_status_async(workspace: *const c_void, code_dst: *mut i32, cuda_stream: *mut c_void) -> i32;
    pub fn ssd_status_check(code: i32) -> i32;
    pub fn ssd_noalloc_status(cuda_stream: *mut c_void, code_out: *mut i32) -> i32;
    pub fn ssd_launch_count() -> i64;
    pub fn ssd_profile_begin(cuda_stream: *mut c_void) -> i32;
    /// `names`, `ms`: HOST buffers.
    pub fn ssd_profile_end(names: *mut c_char, names_bytes: size_t, ms: *mut f32, max_entries: i32) -> i32;
    pub fn ssd_version() -> i32;
    pub fn ssd_compiled_arch() -> i32;
}

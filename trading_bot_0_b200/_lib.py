"""ctypes binding of the C ABI declared in include/ssd_b200.h.

The structures below mirror the header field for field; this is the same raw-pointer contract a
Rust `extern "C"` block over tch tensors would use (`at_data_ptr`,
vendor/torch-sys-0.25.0/libtch/torch_api.h:41).  There is no CPU or eager fallback: if the
compiled library is missing the import fails loudly.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

# SSD_B200_LIB overrides the library location (e.g. to test a differently built copy).
LIB_PATH = Path(os.environ.get("SSD_B200_LIB") or (Path(__file__).resolve().parent / "lib" / "libssd_b200.so"))

SSD_F32, SSD_BF16 = 0, 1
PASS_FWD, PASS_BWD = 0, 1
ALGO_AUTO, ALGO_FP32_CORES, ALGO_TENSOR, ALGO_TENSOR_ONETILE = 0, 1, 2, 3
STAGE_LOCAL, STAGE_TOTAL, STAGE_FINISH, STAGE_LOCAL_STATES, STAGE_LOCAL_REST = 1, 2, 4, 8, 16
SP_UNIQUE_ID_BYTES = 128

EXPORTS = [
    "ssd_workspace_bytes", "ssd_forward", "ssd_backward", "ssd_forward_staged", "ssd_backward_staged",
    "ssd_state_update", "ssd_state_reset_rows", "ssd_sp_total_logdecay", "ssd_sp_prefix_state",
    "ssd_last_error", "ssd_version", "ssd_compiled_arch", "ssd_launch_count", "ssd_profile_begin",
    "ssd_profile_end", "ssd_forward_noalloc", "ssd_noalloc_max_bytes",
    "ssd_conv1d_workspace_bytes", "ssd_conv1d_forward", "ssd_conv1d_backward",
    "ssd_rmsnorm_workspace_bytes", "ssd_rmsnorm_forward", "ssd_rmsnorm_backward", "ssd_selftest_bounded_wait",
    "ssd_workspace_status", "ssd_workspace_status_async", "ssd_status_check", "ssd_noalloc_status",
    "ssd_sp_unique_id", "ssd_sp_comm_new", "ssd_sp_comm_wrap", "ssd_sp_comm_world", "ssd_sp_comm_rank", "ssd_sp_comm_free",
    "ssd_sp_comm_abort", "ssd_sp_exchange_bytes", "ssd_sp_exchange_fwd", "ssd_sp_exchange_bwd", "ssd_sp_allreduce_params",
]


class SsdDims(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("batch", "seqlen", "nheads", "headdim", "dstate", "ngroups", "chunk",
                                         "dtype", "algo", "device", "has_z", "dt_softplus")] + \
               [(n, C.c_int64) for n in ("x_stride_b", "x_stride_l", "dt_stride_b", "dt_stride_l",
                                         "b_stride_b", "b_stride_l", "c_stride_b", "c_stride_l",
                                         "z_stride_b", "z_stride_l", "y_stride_b", "y_stride_l")]


class SsdFwdPtrs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("x", "dt", "A", "Bm", "Cm", "D", "z", "init_state", "y", "final_state",
                                          "dt_bias")]


class SsdBwdPtrs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("x", "dt", "A", "Bm", "Cm", "D", "z", "init_state", "dy",
                                          "dfinal_state", "dx", "ddt", "dA", "dB", "dC", "dD", "dz",
                                          "dinit_state")] + [("fwd_saved", C.c_int32), ("dt_bias", C.c_void_p),
                                                           ("ddt_bias", C.c_void_p)]


class SsdStepDims(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("streams", "nheads", "headdim", "dstate", "ngroups", "dtype", "device",
                                         "dt_softplus")] + \
               [(n, C.c_int64) for n in ("x_stride_s", "dt_stride_s", "b_stride_s", "c_stride_s", "z_stride_s",
                                         "y_stride_s")]


class SsdStepPtrs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("state", "x", "dt", "A", "Bm", "Cm", "D", "z", "y", "dt_bias")]


class SsdConvDims(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("batch", "seqlen", "channels", "width", "dtype", "device", "activation",
                                         "reserved")] + \
               [(n, C.c_int64) for n in ("in_stride_b", "in_stride_l", "out_stride_b", "out_stride_l")]


class SsdConvGrad(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("channels", C.c_int32), ("reserved", C.c_int32), ("stride_b", C.c_int64),
                ("stride_l", C.c_int64)]


class SsdNormDims(C.Structure):
    _fields_ = [("rows", C.c_int64), ("width", C.c_int32), ("dtype", C.c_int32), ("device", C.c_int32), ("eps", C.c_float),
                ("in_stride_row", C.c_int64), ("out_stride_row", C.c_int64)]


class SsdError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"ssd_b200 error {code}: {msg}")
        self.code = code


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built "
            "(run `python -m trading_bot_0_b200.build`). There is no CPU fallback.")
    lib = C.CDLL(str(LIB_PATH))
    vp, i32, i64, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t
    lib.ssd_workspace_bytes.restype = sz
    lib.ssd_workspace_bytes.argtypes = [C.POINTER(SsdDims), i32]
    for name in ("ssd_forward", "ssd_backward"):
        f = getattr(lib, name)
        f.restype = i32
        f.argtypes = [C.POINTER(SsdDims), vp, vp, sz, vp]
    lib.ssd_forward.argtypes = [C.POINTER(SsdDims), C.POINTER(SsdFwdPtrs), vp, sz, vp]
    lib.ssd_backward.argtypes = [C.POINTER(SsdDims), C.POINTER(SsdBwdPtrs), vp, sz, vp]
    lib.ssd_forward_staged.restype = i32
    lib.ssd_forward_staged.argtypes = [C.POINTER(SsdDims), C.POINTER(SsdFwdPtrs), vp, sz, vp, i32]
    lib.ssd_backward_staged.restype = i32
    lib.ssd_backward_staged.argtypes = [C.POINTER(SsdDims), C.POINTER(SsdBwdPtrs), vp, sz, vp, i32]
    lib.ssd_state_update.restype = i32
    lib.ssd_state_update.argtypes = [C.POINTER(SsdStepDims), C.POINTER(SsdStepPtrs), vp]
    lib.ssd_state_reset_rows.restype = i32
    lib.ssd_state_reset_rows.argtypes = [vp, i64, vp, i64, i64, vp]
    lib.ssd_sp_total_logdecay.restype = i32
    lib.ssd_sp_total_logdecay.argtypes = [C.POINTER(SsdDims), vp, sz, vp, vp]
    lib.ssd_sp_prefix_state.restype = i32
    lib.ssd_sp_prefix_state.argtypes = [vp, vp, i32, i32, i32, i64, i64, vp, vp, vp]
    lib.ssd_last_error.restype = C.c_char_p
    lib.ssd_last_error.argtypes = []
    lib.ssd_launch_count.restype = i64
    lib.ssd_launch_count.argtypes = []
    lib.ssd_profile_begin.restype = i32
    lib.ssd_profile_begin.argtypes = [vp]
    lib.ssd_profile_end.restype = i32
    lib.ssd_profile_end.argtypes = [C.c_char_p, sz, C.POINTER(C.c_float), i32]
    lib.ssd_forward_noalloc.restype = i32
    lib.ssd_forward_noalloc.argtypes = [C.POINTER(SsdDims), C.POINTER(SsdFwdPtrs), vp]
    lib.ssd_noalloc_max_bytes.restype = sz
    lib.ssd_noalloc_max_bytes.argtypes = []
    lib.ssd_selftest_bounded_wait.restype = i32
    lib.ssd_selftest_bounded_wait.argtypes = [vp, i64, vp]
    lib.ssd_sp_unique_id.restype = i32
    lib.ssd_sp_unique_id.argtypes = [vp]
    lib.ssd_sp_comm_new.restype = vp
    lib.ssd_sp_comm_new.argtypes = [vp, i32, i32]
    lib.ssd_sp_comm_wrap.restype = vp
    lib.ssd_sp_comm_wrap.argtypes = [vp]
    for name in ("ssd_sp_comm_world", "ssd_sp_comm_rank", "ssd_sp_comm_abort"):
        getattr(lib, name).restype = i32
        getattr(lib, name).argtypes = [vp]
    lib.ssd_sp_comm_free.restype = None
    lib.ssd_sp_comm_free.argtypes = [vp]
    lib.ssd_sp_exchange_bytes.restype = sz
    lib.ssd_sp_exchange_bytes.argtypes = [C.POINTER(SsdDims), i32]
    for name in ("ssd_sp_exchange_fwd", "ssd_sp_exchange_bwd"):
        getattr(lib, name).restype = i32
        getattr(lib, name).argtypes = [C.POINTER(SsdDims), vp, sz, vp, vp, vp, vp, vp, sz, vp, i32]
    lib.ssd_sp_allreduce_params.restype = i32
    lib.ssd_sp_allreduce_params.argtypes = [vp, vp, vp, i32, vp, i32]
    lib.ssd_workspace_status.restype = i32
    lib.ssd_workspace_status.argtypes = [vp, vp, C.POINTER(i32)]
    lib.ssd_workspace_status_async.restype = i32
    lib.ssd_workspace_status_async.argtypes = [vp, vp, vp]
    lib.ssd_status_check.restype = i32
    lib.ssd_status_check.argtypes = [i32]
    lib.ssd_noalloc_status.restype = i32
    lib.ssd_noalloc_status.argtypes = [vp, C.POINTER(i32)]
    lib.ssd_conv1d_workspace_bytes.restype = sz
    lib.ssd_conv1d_workspace_bytes.argtypes = [C.POINTER(SsdConvDims)]
    lib.ssd_conv1d_forward.restype = i32
    lib.ssd_conv1d_forward.argtypes = [C.POINTER(SsdConvDims), vp, vp, vp, vp, vp]
    lib.ssd_conv1d_backward.restype = i32
    lib.ssd_conv1d_backward.argtypes = [C.POINTER(SsdConvDims), vp, vp, vp, C.POINTER(SsdConvGrad), i32, vp, i64, i64, vp, vp,
                                        vp, sz, vp]
    lib.ssd_rmsnorm_workspace_bytes.restype = sz
    lib.ssd_rmsnorm_workspace_bytes.argtypes = [C.POINTER(SsdNormDims)]
    lib.ssd_rmsnorm_forward.restype = i32
    lib.ssd_rmsnorm_forward.argtypes = [C.POINTER(SsdNormDims), vp, vp, vp, vp, vp]
    lib.ssd_rmsnorm_backward.restype = i32
    lib.ssd_rmsnorm_backward.argtypes = [C.POINTER(SsdNormDims), vp, vp, vp, vp, i64, vp, i64, vp, vp, sz, vp]
    lib.ssd_version.restype = i32
    lib.ssd_compiled_arch.restype = i32
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != 0:
        raise SsdError(rc, load().ssd_last_error().decode("utf-8", "replace"))


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(load().ssd_launch_count())


class profile:
    """Context manager: per-kernel device times (ms) of every library launch made inside it from
    this thread.  `.entries` is a list of (kernel name, ms) in launch order."""

    def __init__(self, stream_ptr: int):
        self.stream_ptr = stream_ptr
        self.entries = []

    def __enter__(self):
        check(load().ssd_profile_begin(C.c_void_p(self.stream_ptr)))
        return self

    def __exit__(self, *exc):
        names = C.create_string_buffer(1 << 16)
        ms = (C.c_float * 256)()
        n = load().ssd_profile_end(names, len(names), ms, 256)
        if n < 0:
            check(n)
        self.entries = list(zip(names.value.decode().split("\n")[:n], [float(ms[i]) for i in range(n)]))
        return False

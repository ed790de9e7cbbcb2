"""The C-ABI library builds, loads and exports every symbol the header declares; argument
validation that needs no device is exercised (no compute call without a GPU)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "ssd_b200.h")).read()
    return sorted(set(re.findall(r"SSD_API\s+[\w\s\*]+?\b(ssd_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from trading_bot_0_b200 import _lib
    syms = header_symbols()
    assert len(syms) >= 12
    assert set(syms) == set(_lib.EXPORTS)
    for s in syms:
        assert getattr(lib, s) is not None, s
    assert lib.ssd_compiled_arch() == 100


def test_struct_sizes_match_header(lib):
    from trading_bot_0_b200 import _lib
    assert C.sizeof(_lib.SsdDims) == 12 * 4 + 12 * 8
    assert C.sizeof(_lib.SsdFwdPtrs) == 11 * 8
    assert C.sizeof(_lib.SsdBwdPtrs) == 18 * 8 + 8 + 2 * 8
    assert C.sizeof(_lib.SsdStepDims) == 8 * 4 + 6 * 8
    assert C.sizeof(_lib.SsdStepPtrs) == 10 * 8


def _dims(**kw):
    from trading_bot_0_b200 import _lib
    d = _lib.SsdDims()
    d.batch, d.seqlen, d.nheads, d.headdim, d.dstate, d.ngroups, d.chunk = 4, 256, 4, 32, 16, 1, 64
    d.device = -1
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def test_workspace_sizes(lib):
    d = _dims()
    fwd = lib.ssd_workspace_bytes(C.byref(d), 0)
    bwd = lib.ssd_workspace_bytes(C.byref(d), 1)
    assert 0 < fwd < bwd and fwd % 256 == 0
    dz = _dims(has_z=1)
    assert lib.ssd_workspace_bytes(C.byref(dz), 1) > bwd


@pytest.mark.parametrize("kw,needle", [({"chunk": 512}, "chunk"), ({"ngroups": 3}, "multiple of ngroups"),
                                       ({"batch": 0}, "positive"), ({"dtype": 9}, "dtype"),
                                       ({"x_stride_l": 7}, "strides")])
def test_invalid_dims_are_rejected_with_a_message(lib, kw, needle):
    d = _dims(**kw)
    assert lib.ssd_workspace_bytes(C.byref(d), 0) == 0
    assert needle in lib.ssd_last_error().decode()


def test_null_pointers_are_rejected_before_any_launch(lib):
    from trading_bot_0_b200 import _lib
    d = _dims()
    p = _lib.SsdFwdPtrs()
    assert lib.ssd_forward(C.byref(d), C.byref(p), None, 0, None) == -6
    assert "non-NULL" in lib.ssd_last_error().decode()
    assert lib.ssd_forward(None, C.byref(p), None, 0, None) == -6
    sd, sp = _lib.SsdStepDims(), _lib.SsdStepPtrs()
    assert lib.ssd_state_update(C.byref(sd), C.byref(sp), None) == -1
    assert lib.ssd_state_reset_rows(None, 8, None, 0, 1, None) == -6
    assert lib.ssd_sp_prefix_state(None, None, 2, 0, 1, 1, 1, None, None, None) == -6


def test_misaligned_pointer_returns_bad_alignment_without_a_launch(lib):
    """Tensor-core family, an output pointer 8 bytes off a 16-byte boundary: refused on the host (nothing is launched, so
    this runs without a GPU); the same pointers pass for the CUDA-core family up to the launch itself, which is not made."""
    from trading_bot_0_b200 import _lib
    d = _dims(seqlen=128, nheads=8, headdim=32, dstate=64, chunk=128, dtype=_lib.SSD_BF16, algo=_lib.ALGO_TENSOR)
    need = lib.ssd_workspace_bytes(C.byref(d), 0)
    assert need > 0
    base = 0x7f0000000000
    p = _lib.SsdFwdPtrs(*[C.c_void_p(base + i * 0x1000000) for i in range(5)], None, None, None, C.c_void_p(base + 0x9000008),
                        None, None)
    rc = lib.ssd_forward(C.byref(d), C.byref(p), C.c_void_p(base + 0xa000000), need, None)
    assert rc == -2 and "y must be 16-byte aligned" in lib.ssd_last_error().decode()


def test_status_word_mapping_needs_no_device(lib):
    assert lib.ssd_status_check(0) == 0
    assert lib.ssd_status_check(47) == -7
    assert "47" in lib.ssd_last_error().decode()


def test_host_side_validation_raises_without_a_gpu():
    import torch
    import trading_bot_0_b200 as T
    x = torch.zeros(1, 8, 2, 4)
    with pytest.raises(ValueError, match="CUDA tensor"):
        T.forward(x, x[..., 0], torch.zeros(2), x, x, chunk=8)
    with pytest.raises(ValueError, match="CUDA tensor"):
        T.state_update(torch.zeros(1, 2, 4, 4), x[0, 0], x[0, 0, :, 0], torch.zeros(2), x[0, :1], x[0, :1])

"""The libtorch autograd node library builds, loads, registers its operators and exports the C entry points a tch-rs
binding would declare; a call with CPU tensors is refused (no compute without a GPU)."""
import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_c_entry_points_are_exported(torch_node_lib):
    src = open(os.path.join(ROOT, "trading_bot_0_b200", "csrc", "ssd_torch.cpp")).read()
    declared = sorted(set(re.findall(r'visibility\("default"\)\)\)\s+[\w\*]+\s+(\w+)\(', src)))
    assert declared == ["atg_ssd_scan", "atg_ssd_state_update", "ssd_torch_get_and_reset_last_err"]
    from trading_bot_0_b200 import torch_node
    torch_node.load()
    h = C.CDLL(str(torch_node_lib))
    for name in declared:
        assert getattr(h, name) is not None


def test_operators_are_registered_with_the_documented_schema(torch_node_lib):
    from trading_bot_0_b200 import torch_node
    torch_node.load()
    s = str(torch.ops.ssd_b200.scan.default._schema)
    assert "Tensor? dt_bias, int chunk, bool dt_softplus, int algo) -> (Tensor, Tensor)" in s
    s = str(torch.ops.ssd_b200.state_update.default._schema)
    assert "Tensor(a!) state" in s and s.endswith("-> Tensor")


def test_cpu_tensors_are_refused(torch_node_lib):
    from trading_bot_0_b200 import torch_node
    x, dt, A, B = torch.zeros(1, 8, 2, 8), torch.zeros(1, 8, 2), torch.zeros(2), torch.zeros(1, 8, 1, 16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        torch_node.ssd_scan(x, dt, A, B, B, chunk=8)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        torch_node.state_update(torch.zeros(2, 2, 8, 16), x[0, :2], dt[0, :2], A, B[0, :2], B[0, :2])


def test_error_messages_with_numbers_format_correctly(torch_node_lib):
    """A message that formats integers and shapes goes through the C++ stream classes inside the library: this crashed the
    process when the library carried a second, static copy of the C++ runtime (the build now links the shared one only)."""
    from trading_bot_0_b200 import torch_node
    x3, dt, A, B = torch.zeros(8, 2, 8), torch.zeros(1, 8, 2), torch.zeros(2), torch.zeros(1, 8, 1, 16)
    with pytest.raises(RuntimeError, match=r"got 3 dims: \[8, 2, 8\]"):
        torch_node.ssd_scan(x3, dt, A, B, B, chunk=8)
    import subprocess
    from trading_bot_0_b200 import build
    syms = subprocess.run(["nm", "-D", "--defined-only", str(build.TORCH_LIB)], capture_output=True, text=True).stdout
    assert "_ZNSo" not in syms and "_ZNSt6locale" not in syms, "the library must not export its own copy of libstdc++"

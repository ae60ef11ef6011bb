"""The C-ABI shared library loads on a CPU-only machine and exports every symbol the header declares."""
import ctypes as C
import os
import re

import pytest

from trigrad_b200 import _native as N
from trigrad_b200 import build as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "trigrad_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tg_[a-z0-9_]+)\s*\(", text)))


def test_library_is_built_and_loads():
    B.build()
    assert os.path.exists(N.LIB_PATH)
    assert N.lib().tg_version() >= 1


def test_every_declared_symbol_is_exported_and_bound():
    lib = C.CDLL(N.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in N.SIGNATURES, f"{name} has no ctypes signature"
    assert set(N.SIGNATURES) == set(names)


def test_status_strings():
    lib = N.lib()
    assert lib.tg_status_string(0) == b"ok"
    for code in range(1, 6):
        assert lib.tg_status_string(code) not in (b"ok", b"unknown status")


def test_argument_errors_are_reported_before_any_device_work():
    lib = N.lib()
    # tile larger than 1024 threads
    st = lib.tg_blend_forward(None, None, None, None, 64, 64, 64, 64, 0.0, 1, 32, None, None, None, None, None, None)
    assert st == N.TG_ERR_BAD_ARG and b"1024" in lib.tg_last_error()
    # max_layers must be >= 1 at the ABI (the Python layer maps <= 0 to T + 1)
    st = lib.tg_blend_forward(None, None, None, None, 64, 64, 16, 16, 0.0, 1, 0, None, None, None, None, None, None)
    assert st == N.TG_ERR_BAD_ARG
    # bad bit range for the sort
    st = lib.tg_sort_pairs(None, None, None, None, 10, 8, 8, None, 0, None, None, None)
    assert st == N.TG_ERR_BAD_ARG
    with pytest.raises(N.NativeError):
        N.check("sort", st)


def test_scratch_size_queries():
    lib = N.lib()
    assert lib.tg_scan_scratch_bytes(0) >= 8
    assert lib.tg_scan_scratch_bytes(10_000_000) > lib.tg_scan_scratch_bytes(1000)
    assert lib.tg_sort_scratch_bytes(1 << 20) > lib.tg_sort_scratch_bytes(1)
    assert lib.tg_backward_scratch_bytes(1000) >= 32 * 1000
    # saved per-pixel selection: only in per-pixel mode with at most one batch of 32 layers
    assert lib.tg_selection_planes(1, 32) == 32 and lib.tg_selection_planes(1, 7) == 7
    assert lib.tg_selection_planes(1, 33) == 0 and lib.tg_selection_planes(0, 32) == 0
    a = lib.tg_forward_workspace_bytes(1000, 64, 5000)
    b = lib.tg_forward_workspace_bytes(1000, 64, 50000)
    assert b > a > 0

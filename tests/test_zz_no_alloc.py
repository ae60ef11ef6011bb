"""The allocation-free scan entry point (``tg_scan_static``) against the regular one (``tg_scan``).

Collected last on purpose (file name), so that a run stopping at the first failure has already run
every other test.  ``tg_scan_static`` serves callers that may not allocate device memory where they
need a scan - a host with a fixed memory plan, a loop that must stay clear of the allocator, a plugin
inside an application that owns all allocations: its scratch is a fixed array inside the library.
Two calls in a row (different sizes, the second smaller) check that what the first call left in the
shared array does not leak into the second.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from trigrad_b200 import _native as N

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _scan_regular(x):
    n = x.numel()
    out = torch.empty(n + 1, dtype=torch.int32, device="cuda")
    nb = N.lib().tg_scan_scratch_bytes(n)
    scratch = torch.empty(nb + 16, dtype=torch.uint8, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    N.check("scan", N.lib().tg_scan(_ptr(x), _ptr(out), n, _ptr(scratch), nb, _ptr(status), _stream()))
    return out, status


def _scan_static(x):
    n = x.numel()
    out = torch.empty(n + 1, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    N.check("scan_static", N.lib().tg_scan_static(_ptr(x), _ptr(out), n, _ptr(status), _stream()))
    return out, status


def test_static_scan_matches_regular_scan_on_two_calls_in_a_row():
    rng = np.random.default_rng(42)
    for n in (3_000_001, 70_000):          # second call smaller: stale words of the first must not matter
        x = torch.from_numpy(rng.integers(0, 40, n, dtype=np.int32)).cuda()
        ref, st_ref = _scan_regular(x)
        got, st_got = _scan_static(x)
        torch.cuda.synchronize()
        assert int(st_ref[0]) == 0 and int(st_got[0]) == 0
        assert torch.equal(got, ref)       # integer work: exact
        assert int(got[-1]) == int(x.sum())


def test_static_scan_at_its_largest_size():
    """n = 2^24 is the one size that uses the last word of the fixed array."""
    n = 1 << 24
    x = torch.from_numpy(np.random.default_rng(1).integers(0, 100, n, dtype=np.int32)).cuda()
    ref, _ = _scan_regular(x)
    got, st = _scan_static(x)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    assert torch.equal(got, ref)


def test_static_scan_leaves_free_device_memory_unchanged():
    """The property in the entry point's name: with outputs allocated beforehand, a call changes neither the
    driver's figure of free device memory nor the figures of torch's caching allocator."""
    n = 1_000_000
    x = torch.ones(n, dtype=torch.int32, device="cuda")
    out = torch.empty(n + 1, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    lib = N.lib()
    N.check("scan_static", lib.tg_scan_static(_ptr(x), _ptr(out), n, _ptr(status), _stream()))   # first call: address look-up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    reserved0, allocated0 = torch.cuda.memory_reserved(), torch.cuda.memory_allocated()
    N.check("scan_static", lib.tg_scan_static(_ptr(x), _ptr(out), n, _ptr(status), _stream()))
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert torch.cuda.memory_reserved() == reserved0 and torch.cuda.memory_allocated() == allocated0
    assert int(out[-1]) == n and int(status[0]) == 0


def test_static_scan_rejects_sizes_beyond_its_fixed_array():
    n = (1 << 24) + 1
    x = torch.zeros(n, dtype=torch.int32, device="cuda")
    out = torch.empty(n + 1, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    st = N.lib().tg_scan_static(_ptr(x), _ptr(out), n, _ptr(status), _stream())
    assert st == N.TG_ERR_CAPACITY
    assert b"at most" in N.lib().tg_last_error()

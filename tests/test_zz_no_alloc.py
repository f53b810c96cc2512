"""rh_selftest_static — the self-check for hosts that cannot use the device allocator any more (an
engine that gave all of HBM to its arenas and KV cache at start-up: cudaMalloc may fail there and
stalls the device when it works).  Its counters live in a fixed array inside the library instead of
a cudaMalloc'ed buffer, so the array still holds the previous call's values when the next call starts.
Called through the C ABI twice in a row, it must report exactly what the allocating rh_selftest
reports (integer counts: no tolerance), and must refuse more counters than the array has.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.  It must also pass when run alone in a fresh process (the first call does the set-up)."""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu


def test_static_selftest_matches_allocating_selftest_twice():
    import torch
    from runtherder_b200 import _lib
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    want = (C.c_uint * 8)()
    _lib.call("rh_selftest", want)
    want = list(want)
    stream = torch.cuda.Stream()
    for attempt in range(2):                       # the second call meets the first call's leftovers
        for n in (8, 6, 3):
            got = (C.c_uint * 8)(*([0xDEADBEEF] * 8))
            _lib.call("rh_selftest_static", got, n, stream.cuda_stream)
            assert list(got)[:n] == want[:n], (attempt, n, list(got), want)
            assert all(v == 0xDEADBEEF for v in list(got)[n:])     # nothing written past num_counters
    got = (C.c_uint * 8)()
    _lib.call("rh_selftest_static", got, 8, None)                  # legacy default stream
    assert list(got) == want
    assert want[0] == 0 and want[1] == 0 and want[2:6] == [0, 0, 0, 0]


def test_static_selftest_rejects_oversize_and_bad_arguments():
    from runtherder_b200 import _lib
    buf = (C.c_uint * 16)()
    assert _lib.lib.rh_selftest_static(buf, 9, None) == 2          # RH_ERR_UNSUPPORTED_DIM
    assert b"exceeds the fixed scratch of 8" in _lib.lib.rh_last_error_string()
    assert _lib.lib.rh_selftest_static(buf, 0, None) == 1
    assert _lib.lib.rh_selftest_static(None, 4, None) == 1

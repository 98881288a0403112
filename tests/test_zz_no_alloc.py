"""b200_reduce_all_static: the whole-tensor reduction for callers that must not allocate.

Such callers (a serving loop that has given all device memory to its own pools, a latency-bound
thread that may not take the driver's allocation lock, a process with a memory budget fixed at
start-up) cannot use b200_reduce_all, which reserves its scratch with cudaMalloc on first use.
This entry point keeps that scratch in a fixed array inside the library. The test drives it
through the C ABI twice in a row (the array keeps the previous call's contents, so the second
call checks that what must start at zero is cleared) and compares with b200_reduce_all.

Collected last on purpose: a failure here must not keep any other test from running.
"""
import ctypes as C

import numpy as np
import pytest

from gorgonia_b200 import _lib
from gorgonia_b200._lib import lib
from tests import util

pytestmark = pytest.mark.gpu


def _reduce(fn, e, kind, tx, ty):
    rc = fn(e.h, _lib.F32 if tx.dtype == np.float32 else _lib.F64, kind, tx.ptr, tx.size, ty.ptr)
    assert rc == 0, lib.b200_last_error(e.h)
    return ty.numpy()[0]


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_static_scratch_reduction_matches_allocating_one(dt):
    from gorgonia_b200 import Engine
    e = Engine(0, 64 << 20)
    try:
        for n in (1, 1000, 300_007, 2_000_003):
            x = util.normal(17 + n, n, dt)
            tx, y_ref, y_new = e.tensor(x), e.empty(1, dt), e.empty(1, dt)
            scale = float(np.abs(x.astype(np.float64)).sum())
            tol = (1e-6 if dt == np.float32 else 1e-14) * scale     # the sums' tolerance elsewhere
            for kind in (0, 1):
                want = _reduce(lib.b200_reduce_all, e, kind, tx, y_ref)
                for call in range(2):                                # two calls in a row
                    got = _reduce(lib.b200_reduce_all_static, e, kind, tx, y_new)
                    if kind == 1:
                        assert got == want == x.max()
                    else:
                        assert abs(float(got) - float(want)) <= tol, (n, call, got, want)
                        assert abs(float(got) - float(np.sum(x.astype(np.float64)))) <= tol
            for t in (tx, y_ref, y_new):
                t.free()
    finally:
        e.Close()


def test_static_scratch_reduction_refuses_oversize():
    from gorgonia_b200 import Engine
    e = Engine(0, 1 << 20)
    try:
        x, y = e.empty(4), e.empty(1)
        rc = lib.b200_reduce_all_static(e.h, _lib.F32, 0, x.ptr, (1 << 32) + 1, y.ptr)
        assert rc == _lib.ERR_UNSUPPORTED
        assert b"exceed the limit" in lib.b200_last_error(e.h)
    finally:
        e.Close()

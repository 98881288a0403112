"""CPU-only checks of the C ABI: the library loads, exports what the header declares, and the
host-side parts that need no device (allocator, fusion planner) behave as specified."""
import ctypes as C

import pytest

from gorgonia_b200 import _lib
from gorgonia_b200._lib import lib


def test_library_exports_every_declared_symbol():
    names = _lib.declared_symbols()
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(lib, n)]
    assert missing == []


def test_every_declared_symbol_has_a_python_signature():
    unbound = [n for n in _lib.declared_symbols() if n not in _lib._SIGS]
    assert unbound == []


def test_engine_create_without_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = lib.b200_engine_create(0, 1 << 20, 0, C.byref(h))
    assert rc != _lib.OK and not h.value
    assert lib.b200_last_error(None)


# ---- allocator: the contract gorgonia's cuda/bfc_test.go:47-120 checks ----------------------

def _alloc(a, n):
    off = C.c_int64(-1)
    rc = lib.b200_bfc_alloc(a, n, C.byref(off))
    return rc, off.value


def test_bfc_contract():
    align = 32
    a = lib.b200_bfc_create(1024, align)
    try:
        rc, _ = _alloc(a, 0)
        assert rc == _lib.ERR_INVALID            # alloc(0) is an error
        rc, addr0 = _alloc(a, 21)                 # smaller than the alignment
        assert rc == 0 and addr0 % align == 0
        assert lib.b200_bfc_free_blocks(a) == 1
        rc, addr1 = _alloc(a, align)              # exactly the alignment
        assert rc == 0 and addr1 % align == 0 and addr1 != addr0
        rc, addr2 = _alloc(a, 69)                 # larger than the alignment
        assert rc == 0 and addr2 % align == 0
        assert lib.b200_bfc_used(a) == 32 + 32 + 96
        # free in the middle, then reuse the hole
        lib.b200_bfc_free(a, addr1)
        assert lib.b200_bfc_free_blocks(a) == 2
        rc, addr3 = _alloc(a, 20)
        assert rc == 0 and addr3 == addr1
        # freeing an unknown address changes nothing
        used = lib.b200_bfc_used(a)
        lib.b200_bfc_free(a, 7)
        assert lib.b200_bfc_used(a) == used
        # out of memory is reported, not fatal
        rc, _ = _alloc(a, 4096)
        assert rc == _lib.ERR_OOM
        # freeing everything coalesces back to one block
        for off in (addr0, addr2, addr3):
            lib.b200_bfc_free(a, off)
        assert lib.b200_bfc_free_blocks(a) == 1
        assert lib.b200_bfc_largest_free(a) == 1024 and lib.b200_bfc_used(a) == 0
    finally:
        lib.b200_bfc_destroy(a)


def test_bfc_fragmentation_and_reset():
    a = lib.b200_bfc_create(256 * 16, 256)
    try:
        offs = [_alloc(a, 256)[1] for _ in range(16)]
        assert sorted(offs) == [256 * i for i in range(16)]
        assert _alloc(a, 1)[0] == _lib.ERR_OOM
        for o in offs[::2]:
            lib.b200_bfc_free(a, o)
        assert lib.b200_bfc_free_blocks(a) == 8 and lib.b200_bfc_largest_free(a) == 256
        assert _alloc(a, 512)[0] == _lib.ERR_OOM          # fragmented: no 512-byte hole
        lib.b200_bfc_free(a, offs[1])                       # joins holes 0,1,2
        assert lib.b200_bfc_largest_free(a) == 768
        assert _alloc(a, 512) == (0, 0)
        lib.b200_bfc_reset(a)
        assert lib.b200_bfc_used(a) == 0 and lib.b200_bfc_free_blocks(a) == 1
    finally:
        lib.b200_bfc_destroy(a)


# ---- fusion planner ----------------------------------------------------------------------

def _call(op, dst, a=0, b=0, form=_lib.VV, n=1024, dtype=_lib.F32, scalar=0.0, bcast=0, bdiv=0, bmod=0):
    c = _lib.PwCall()
    c.op, c.dtype, c.form, c.bcast = _lib.OP[op], dtype, form, bcast
    c.dst, c.a, c.b, c.scalar, c.n, c.bdiv, c.bmod = dst, a, b, scalar, n, bdiv, bmod
    return c


def _plan(calls, released=None):
    n = len(calls)
    arr = (_lib.PwCall * n)(*calls)
    rel = (C.c_int * n)(*(released or [-1] * n))
    koc = (C.c_int * n)()
    loads = (C.c_int * n)()
    stores = (C.c_int * n)()
    nk = C.c_int()
    assert lib.b200_fusion_plan(arr, n, rel, koc, C.byref(nk), loads, stores) == 0
    return list(koc), nk.value, list(loads)[:nk.value], list(stores)[:nk.value]


X, W, Bb, T1, T2, T3 = (0x10000 * k for k in range(1, 7))
UN = 3


def test_plan_in_place_chain_is_one_kernel():
    # x = x*w ; x = x+b ; x = tanh(x)   (the reference would launch 3 kernels)
    calls = [_call("mul", X, X, W), _call("add", X, X, Bb), _call("tanh", X, X, form=UN)]
    koc, nk, loads, stores = _plan(calls)
    assert nk == 1 and koc == [0, 0, 0]
    assert loads == [3] and stores == [1]


def test_plan_released_intermediates_are_not_stored():
    calls = [_call("mul", T1, X, W), _call("add", T2, T1, Bb), _call("tanh", T3, T2, form=UN)]
    _, nk, loads, stores = _plan(calls)
    assert nk == 1 and loads == [3] and stores == [3]       # nobody released anything: 3 stores
    _, nk, loads, stores = _plan(calls, released=[2, 3, -1])
    assert nk == 1 and loads == [3] and stores == [1]       # T1, T2 handed back before the flush


def test_plan_splits_on_size_dtype_and_overlap():
    calls = [_call("add", T1, X, W), _call("add", T2, X, W, n=512)]
    assert _plan(calls)[1] == 2
    calls = [_call("add", T1, X, W), _call("add", T2, X, W, dtype=_lib.F64)]
    assert _plan(calls)[1] == 2
    # second call reads a buffer that partly overlaps what the first one writes
    calls = [_call("add", T1, X, W), _call("neg", T2, T1 + 64, form=UN)]
    assert _plan(calls)[1] == 2
    # second call writes over part of a buffer the first one reads
    calls = [_call("add", T1, X, W), _call("neg", X + 64, T1, form=UN)]
    assert _plan(calls)[1] == 2


def test_plan_leaky_relu_is_one_kernel():
    # LeakyRelu as gorgonia builds it (nn.go:104-130): 6 instructions, here after a bias add
    P, N, A, R = T1, T2, T3, 0x70000
    calls = [
        _call("add", X, X, Bb, bcast=1, bdiv=1, bmod=256),
        _call("gte", P, X, form=_lib.VS, scalar=0.0),
        _call("lt", N, X, form=_lib.VS, scalar=0.0),
        _call("mul", P, X, P),
        _call("mul", N, X, N),
        _call("mul", N, N, form=_lib.VS, scalar=0.1),
        _call("add", R, P, N),
    ]
    koc, nk, loads, stores = _plan(calls, released=[-1, -1, -1, 7, -1, 7, -1])
    assert nk == 1
    assert loads == [1]
    assert stores == [2]       # x (bias added in place) and the result; P and N were released


def test_plan_limits_program_length():
    calls = [_call("neg", X, X, form=UN) for _ in range(20)]
    koc, nk, _, _ = _plan(calls)
    assert nk == 3 and koc.count(0) == 8

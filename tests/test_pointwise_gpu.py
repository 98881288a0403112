"""Parity of the pointwise engine methods against the CPU oracle (GPU tests, through the C ABI).

Mirrors TestCUDABasicArithmetic / TestCUDACube of gorgonia (op_math_cuda_test.go:16-109): every
op in every operand form, in the reuse and unsafe modes, plus the sizes around the vector
width and block size where indexing bugs live."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle
from tests import util
from tests.util import assert_bits_equal, assert_pointwise_close

pytestmark = pytest.mark.gpu

DTYPES = (np.float32, np.float64)


def _check(op, g, r):
    if op in util.CMP_OPS or op in ("add", "sub", "mul", "div", "abs", "sign", "ceil", "floor", "neg", "square",
                                    "cube", "sqrt", "inv"):
        assert_bits_equal(g, r)       # exactly rounded IEEE operations: nothing to tolerate
    else:
        assert_pointwise_close(g, r)


def _operands(op, seed, n, dt):
    a = util.normal(seed, n, dt)
    b = util.normal(seed + 1, n, dt)
    if op == "pow":
        a = (np.abs(a) + dt(0.1)).astype(dt)
    if op in ("eq", "ne", "lte", "gte"):
        b[::3] = a[::3]               # make equality actually happen
    return a, b


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("op", util.ARITH_OPS + util.CMP_OPS)
def test_binary_vv_reuse_and_unsafe(fresh, op, dt):
    e = fresh
    for n in util.EDGE_SIZES + (1 << 20, util.STREAM_SIZE):
        a, b = _operands(op, 11 + n, n, dt)
        want = oracle.binary(op, a, b)
        ta, tb, tr = e.tensor(a), e.tensor(b), e.empty(n, dt)
        out = getattr(e, {"eq": "ElEq", "ne": "ElNe"}.get(op, op.capitalize()))(ta, tb, reuse=tr)
        assert out is tr
        _check(op, tr.numpy(), want)
        assert_bits_equal(ta.numpy(), a)          # reuse leaves the operands alone
        out = e._binary(op, ta, tb, unsafe=True)  # unsafe overwrites a
        assert out is ta
        _check(op, ta.numpy(), want)
        for t in (ta, tb, tr):
            t.free()


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("op", util.ARITH_OPS + util.CMP_OPS)
def test_binary_scalar_forms(fresh, op, dt):
    e = fresh
    for n in (1, 5, 1025, 65536 + 3, util.STREAM_SIZE):
        a, _ = _operands(op, 7 + n, n, dt)
        s = dt(0.75)
        ta, tr = e.tensor(a), e.empty(n, dt)
        # tensor op scalar
        e._binary_scalar(op, ta, s, leftTensor=True, reuse=tr)
        _check(op, tr.numpy(), oracle.binary(op, a, s))
        # scalar op tensor: the result lands in the tensor's buffer (cuda/arith.go:109-112)
        base = (np.abs(a) + dt(0.1)).astype(dt) if op == "pow" else a
        tb = e.tensor(base)
        sb = dt(1.5)
        e._binary_scalar(op, tb, sb, leftTensor=False, unsafe=True)
        _check(op, tb.numpy(), oracle.binary(op, sb, base))
        # scalar held in device memory, as the reference passes it (cuda/arith.go:73-77)
        ts = e.tensor(np.array([s], dtype=dt))
        e._binary_scalar(op, ta, ts, leftTensor=True, reuse=tr)
        _check(op, tr.numpy(), oracle.binary(op, a, s))
        for t in (ta, tb, tr, ts):
            t.free()


def test_scalar_scalar(fresh):
    # the "ss" form (op_math_cuda.go:139-176): two one-element device buffers
    e = fresh
    for op in ("add", "sub", "mul", "div", "gt"):
        a, b = e.tensor(np.array([3.0], np.float32)), e.tensor(np.array([2.0], np.float32))
        e._binary(op, a, b, unsafe=True)
        assert_bits_equal(a.numpy(), oracle.binary(op, np.array([3.0], np.float32), np.array([2.0], np.float32)))


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("op", util.UNARY_OPS)
def test_unary(fresh, op, dt):
    e = fresh
    for n in util.EDGE_SIZES + (1 << 20, util.STREAM_SIZE):
        x = util.unary_input(op, 3 + n, n, dt)
        if op in ("sigmoid", "softplus") and n >= 1023:
            x[:8] = np.array([-200, -104, -103, -89, -88, 14.5, 15.5, 30], dtype=dt)  # threshold branches
        want = oracle.unary(op, x)
        tx, tr = e.tensor(x), e.empty(n, dt)
        e.Unary(op, tx, reuse=tr)
        _check(op, tr.numpy(), want)
        e.Unary(op, tx, unsafe=True)
        _check(op, tx.numpy(), want)
        tx.free()
        tr.free()


def test_pow_float32_over_the_whole_domain(fresh):
    # the float32 power runs a pair-arithmetic fast path for positive normal bases and hands every
    # other case to the library routine: both, and the hand-over, against the oracle
    e = fresh
    g = util.rng(77)
    n = 1 << 18
    cases = [
        (np.exp(g.uniform(-80, 80, n)), g.uniform(-1.5, 1.5, n)),            # bases over the exponent range
        (np.exp(g.uniform(-3, 3, n)), g.uniform(-45, 45, n)),                 # results up to the ends of the range
        (1 + g.uniform(-2e-3, 2e-3, n), g.uniform(-3e4, 3e4, n)),             # bases next to 1, huge exponents
        (np.exp(g.uniform(-1, 1, n)), np.rint(g.uniform(-8, 8, n))),          # whole exponents
        (g.standard_normal(n), np.rint(g.uniform(-5, 5, n))),                 # negative bases, whole exponents
        (g.standard_normal(n), g.standard_normal(n)),                         # negative bases: NaN where the oracle says so
        (g.uniform(1e-45, 1e-38, n), g.uniform(-1, 1, n)),                    # subnormal bases
    ]
    sp = np.array([0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, np.nan, 2.0, 0.5, 3e-45, 3.4e38, 1.2e-38], dtype=np.float32)
    cases.append((np.repeat(sp, sp.size), np.tile(np.concatenate([sp[:9], np.array([3.0, -3.0, 0.25], np.float32)]), sp.size)))
    for a, b in cases:
        a, b = a.astype(np.float32), b.astype(np.float32)
        with np.errstate(all="ignore"):
            want = oracle.binary("pow", a, b)
        ta, tb, tr = e.tensor(a), e.tensor(b), e.empty(a.size)
        e.Pow(ta, tb, reuse=tr)
        assert_pointwise_close(tr.numpy(), want)
        for t in (ta, tb, tr):
            t.free()


def test_tanh_float32_arms_and_ends(fresh):
    # the polynomial arm, the exponential arm, their seam at 0.55, saturation and special values
    e = fresh
    g = util.rng(78)
    x = np.concatenate([g.uniform(-0.56, 0.56, 1 << 16), g.uniform(0.54, 0.56, 1 << 14), g.uniform(-12, 12, 1 << 16),
                        g.uniform(-100, 100, 1 << 12), np.exp(g.uniform(-60, -3, 1 << 12)),
                        np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 0.55, -0.55, 44.3, 44.5, 3e-45, -1e-38])])
    x = x.astype(np.float32)
    tx = e.tensor(x)
    e.Unary("tanh", tx, unsafe=True)
    got = tx.numpy()
    assert_pointwise_close(got, oracle.unary("tanh", x))
    assert np.signbit(got[x == 0]).tolist() == np.signbit(x[x == 0]).tolist()   # tanh(-0) = -0
    assert (np.abs(got[~np.isnan(x)]) <= 1).all()


def test_sigmoid_float32_both_arms_and_ends(fresh):
    # 1 / (1 + t) above zero, t / (1 + t) below, the thresholds of the reference, results below the
    # normal range, special values
    e = fresh
    g = util.rng(79)
    x = np.concatenate([g.uniform(-20, 20, 1 << 16), g.uniform(-88, -80, 1 << 12), g.uniform(14, 16, 1 << 10),
                        g.standard_normal(1 << 16) * 1e-3,
                        np.array([0.0, -0.0, np.inf, -np.inf, np.nan, -88.0, -87.99, -87.5, -87.3, 15.0, 15.01, 3e-45])])
    x = x.astype(np.float32)
    tx = e.tensor(x)
    e.Unary("sigmoid", tx, unsafe=True)
    assert_pointwise_close(tx.numpy(), oracle.unary("sigmoid", x))


@pytest.mark.parametrize("dt", DTYPES)
def test_single_source_ops_on_wide_tiles(fresh, dt):
    # programs with one full-size source and one instruction run with four 16-byte chunks per thread and tile once
    # every CTA gets several such tiles: a size above that threshold with a ragged last tile and a ragged last
    # chunk, for a unary op, a tensor-scalar op in both operand orders, and the unsafe (in-place) form
    e = fresh
    n = (5 << 22) + 3 if dt == np.float32 else (5 << 21) + 1
    x = util.normal(501, n, dt)
    tx, tr = e.tensor(x), e.empty(n, dt)
    e.Unary("tanh", tx, reuse=tr)
    assert_pointwise_close(tr.numpy(), oracle.unary("tanh", x))
    e.Unary("neg", tx, reuse=tr)
    assert_bits_equal(tr.numpy(), oracle.unary("neg", x))
    s = dt(1.25)
    e._binary_scalar("sub", tx, s, leftTensor=True, reuse=tr)
    assert_bits_equal(tr.numpy(), oracle.binary("sub", x, s))
    e._binary_scalar("sub", tx, s, leftTensor=False, reuse=tr)
    assert_bits_equal(tr.numpy(), oracle.binary("sub", s, x))
    e.Unary("exp", tx, unsafe=True)
    assert_pointwise_close(tx.numpy(), oracle.unary("exp", x))


def test_safe_mode_is_an_error(fresh):
    # cuda/arith.go:47-48: neither reuse nor unsafe -> error
    from gorgonia_b200 import B200Error
    a = fresh.tensor(np.ones(4, np.float32))
    with pytest.raises(B200Error):
        fresh.Add(a, a)


def test_special_values_compare_and_rectify(fresh):
    e = fresh
    x = np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 1.0, -1.0, 3e-45], dtype=np.float32)
    y = np.array([np.nan, np.inf, 1.0, -0.0, 0.0, 1.0, np.nan, 0.0], dtype=np.float32)
    for op in util.CMP_OPS:
        tx, ty = e.tensor(x), e.tensor(y)
        e._binary(op, tx, ty, unsafe=True)
        assert_bits_equal(tx.numpy(), oracle.binary(op, x, y))
    # Rectify = x * (x >= 0) gives -0.0 for negative inputs and NaN for -Inf (nn.go:154-162)
    tx, tm = e.tensor(x), e.empty(8)
    e.GteScalar(tx, 0.0, reuse=tm)
    e.Mul(tx, tm, unsafe=True)
    assert_bits_equal(tx.numpy(), oracle.rectify(x))


def test_unaligned_views(fresh):
    e = fresh
    from gorgonia_b200 import Tensor
    n = 1000
    a, b = util.normal(1, n + 3), util.normal(2, n + 3)
    ta, tb, tr = e.tensor(a), e.tensor(b), e.empty(n + 3)
    va = Tensor(e, ta.ptr + 4, (n,), np.float32, owned=False)
    vb = Tensor(e, tb.ptr + 8, (n,), np.float32, owned=False)
    vr = Tensor(e, tr.ptr + 12, (n,), np.float32, owned=False)
    e.Mul(va, vb, reuse=vr)
    assert_bits_equal(vr.numpy(), a[1:n + 1] * b[2:n + 2])


@pytest.mark.parametrize("dt", DTYPES)
def test_broadcast_forms(fresh, dt):
    e = fresh
    R, Cc = 37, 1024
    a = util.normal(5, (R, Cc), dt)
    row, col = util.normal(6, Cc, dt), util.normal(7, R, dt)
    ta, trow, tcol, tr = e.tensor(a), e.tensor(row), e.tensor(col), e.empty((R, Cc), dt)
    e.BroadcastBinary("add", ta, trow, 1, Cc, reuse=tr)
    assert_bits_equal(tr.numpy(), a + row[None, :])
    e.BroadcastBinary("sub", tcol, ta, Cc, R, bcast_is_a=True, reuse=tr)
    assert_bits_equal(tr.numpy(), col[:, None] - a)
    # odd inner size: falls off the vector path
    R2, C2 = 13, 77
    a2, row2, col2 = util.normal(8, (R2, C2), dt), util.normal(9, C2, dt), util.normal(10, R2, dt)
    t2, tr2 = e.tensor(a2), e.empty((R2, C2), dt)
    e.BroadcastBinary("mul", t2, e.tensor(row2), 1, C2, reuse=tr2)
    assert_bits_equal(tr2.numpy(), a2 * row2[None, :])
    e.BroadcastBinary("div", t2, e.tensor(col2), C2, R2, reuse=tr2)
    assert_bits_equal(tr2.numpy(), a2 / col2[:, None])
    # large enough for the streaming kernel: row operand (vector loads) and column operand
    R3, C3 = 4099, 1024
    a3, row3, col3 = util.normal(13, (R3, C3), dt), util.normal(14, C3, dt), util.normal(15, R3, dt)
    t3, tr3 = e.tensor(a3), e.empty((R3, C3), dt)
    e.BroadcastBinary("add", t3, e.tensor(row3), 1, C3, reuse=tr3)
    assert_bits_equal(tr3.numpy(), a3 + row3[None, :])
    e.BroadcastBinary("mul", e.tensor(col3), t3, C3, R3, bcast_is_a=True, reuse=tr3)
    assert_bits_equal(tr3.numpy(), col3[:, None] * a3)
    # per-channel operand over (B, C, H, W)
    x = util.normal(11, (3, 5, 4, 4), dt)
    ch = util.normal(12, 5, dt)
    tx = e.tensor(x)
    e.BroadcastBinary("add", tx, e.tensor(ch), 16, 5, unsafe=True)
    assert_bits_equal(tx.numpy(), x + ch[None, :, None, None])
    assert_bits_equal(oracle.binary_bcast("add", x, ch, 16, 5), x + ch[None, :, None, None])


@pytest.mark.parametrize("n", [1 << 20, util.STREAM_SIZE, (1 << 23) + 3])
def test_deferred_chain_fuses_into_one_launch(fresh, n):
    e = fresh
    x, w, b = util.normal(1, n), util.normal(2, n), util.normal(3, n)
    tx, tw, tb = e.tensor(x), e.tensor(w), e.tensor(b)
    e.Signal()
    before = e.launches
    e.Mul(tx, tw, unsafe=True)
    e.Add(tx, tb, unsafe=True)
    e.Unary("tanh", tx, unsafe=True)
    assert e.pending() == (3, 1)
    assert e.launches == before            # nothing has been launched yet
    got = tx.numpy()                       # a device-to-host read flushes the queue
    assert e.launches == before + 1
    want = oracle.unary("tanh", oracle.binary("add", oracle.binary("mul", x, w), b))
    assert_pointwise_close(got, want)
    # the unfused engine gives the same bits
    from gorgonia_b200 import Engine
    e2 = Engine(0, 3 * 4 * n + (1 << 20), defer=False)
    ux, uw, ub = e2.tensor(x), e2.tensor(w), e2.tensor(b)
    l0 = e2.launches
    e2.Mul(ux, uw, unsafe=True)
    e2.Add(ux, ub, unsafe=True)
    e2.Unary("tanh", ux, unsafe=True)
    assert e2.launches == l0 + 3
    assert_bits_equal(ux.numpy(), got)
    e2.Close()


def test_released_intermediates_and_leaky_relu(fresh):
    # LeakyRelu exactly as gorgonia's graph spells it (nn.go:104-130), temporaries released
    e = fresh
    n = 3_000_003
    x = util.normal(21, n)
    tx = e.tensor(x)
    e.Signal()
    l0 = e.launches
    p, m = e.empty(n), e.empty(n)
    e.GteScalar(tx, 0.0, reuse=p)
    e.LtScalar(tx, 0.0, reuse=m)
    e.Mul(tx, p, reuse=p)
    e.Mul(tx, m, reuse=m)
    e.MulScalar(m, 0.1, unsafe=True)
    r = e.empty(n)
    e.Add(p, m, reuse=r)
    p.free()
    m.free()
    got = r.numpy()
    assert e.launches == l0 + 1
    assert_bits_equal(got, oracle.leaky_relu(x, 0.1))
    assert_bits_equal(tx.numpy(), x)


def test_explicit_program(fresh):
    from gorgonia_b200._lib import REF_SRC, REF_IMM, REF_INS
    e = fresh
    n = 4097
    x, w = util.normal(1, n), util.normal(2, 64)
    tx, tw, o1, o2 = e.tensor(x), e.tensor(w), e.empty(n), e.empty(n)
    prog = dict(instr=[("mul", REF_SRC(0), REF_SRC(1)), ("add", REF_INS(0), REF_IMM(0)), ("sigmoid", REF_INS(1), 0)],
                imm=[0.5], out=[2, 0], bcast={1: (1, 64)})
    e.Pointwise(prog, [o1, o2], [tx, tw], n)
    t = x * np.tile(w, n // 64 + 1)[:n]
    assert_bits_equal(o2.numpy(), t)
    assert_pointwise_close(o1.numpy(), oracle.unary("sigmoid", t + np.float32(0.5)))


def test_has_nan_has_inf(fresh):
    e = fresh
    x = util.normal(1, 1 << 20)
    t = e.tensor(x)
    assert not e.HasNaN(t) and not e.HasInf(t)
    x[777_777] = np.nan
    t.set(x)
    assert e.HasNaN(t) and not e.HasInf(t)
    x[777_777] = -np.inf
    t.set(x)
    assert e.HasInf(t) and not e.HasNaN(t)


def test_arena_contract_on_device(fresh):
    from gorgonia_b200 import B200Error, Engine
    e = Engine(0, 1 << 20)
    p = e.Get(100)
    assert p % 256 == 0
    with pytest.raises(B200Error) as ei:
        e.Get(0)
    assert ei.value.code == 1
    with pytest.raises(B200Error) as ei:
        e.Get(2 << 20)
    assert ei.value.code == 2 and "out of memory" in ei.value.text
    e.Put(p)
    e.Put(12345)                    # unknown address: silently ignored
    assert e.arena_stats()["used"] == 0
    e.Close()


def test_managed_arena_is_host_readable():
    # gorgonia reads device values from the host (values.go:150-160, vm_tape_cuda.go:139-150)
    from gorgonia_b200 import Engine
    e = Engine(0, 8 << 20, managed=True)
    a = e.tensor(np.arange(8, dtype=np.float32))
    e.AddScalar(a, 1.0, unsafe=True)
    e.Signal()
    host_view = np.ctypeslib.as_array(C.cast(a.ptr, C.POINTER(C.c_float)), shape=(8,))
    assert host_view.tolist() == [1, 2, 3, 4, 5, 6, 7, 8]
    e.Close()


def test_more_than_2_to_the_31_elements():
    # gorgonia's kernels take `int size` (elembinop.cu:8-14): 2^31 elements is out of their reach.
    # Here counts and offsets are 64-bit: a vector of 2^31 + 1027 floats (8.6 GB) goes through the
    # streaming kernel, and the far end, which only a 64-bit index reaches, is read back.
    import ctypes as C
    from gorgonia_b200 import Engine, Tensor
    from gorgonia_b200._lib import lib, check
    n = (1 << 31) + 1027
    e = Engine(0, 2 * 4 * n + (64 << 20))
    try:
        a, b = e.empty(n), e.empty(n)
        check(lib.b200_memset(e.h, a.ptr, 0, 4 * n), e.h)
        e.AddScalar(a, 1.5, unsafe=True)               # a = 1.5 everywhere
        e.MulScalar(a, 2.0, reuse=b)                   # b = 3.0
        e.Unary("neg", b, unsafe=True)                 # b = -3.0, fused with the line above
        tail = Tensor(e, b.ptr + 4 * (n - 2000), (2000,), np.float32, owned=False)
        head = Tensor(e, b.ptr, (2000,), np.float32, owned=False)
        mid = Tensor(e, b.ptr + 4 * ((1 << 31) - 1000), (2000,), np.float32, owned=False)
        for view in (head, mid, tail):
            assert np.all(view.numpy() == np.float32(-3.0))
        s = e.empty(1)
        e.ReduceAll("max", b, s)
        assert s.numpy()[0] == np.float32(-3.0)
    finally:
        e.Close()


def test_empty_inputs_are_no_ops(fresh):
    e = fresh
    from gorgonia_b200._lib import lib, F32, OP, VV
    assert lib.b200_binary(e.h, OP["add"], F32, VV, None, None, None, 0.0, 0, 0) == 0
    assert lib.b200_unary(e.h, OP["exp"], F32, None, None, 0) == 0
    assert lib.b200_softmax(e.h, F32, None, None, 0, 5, 1, 0) == 0
    assert lib.b200_gemm(e.h, F32, 0, 0, 0, 5, 3, None, 3, None, 5, None, 5, 1, 0, 0, 0, None) == 0
    assert lib.b200_transpose(e.h, 4, None, None, 2, (C.c_int64 * 2)(0, 4), (C.c_int * 2)(1, 0)) == 0
    assert lib.b200_gather_rows(e.h, None, None, None, 0, 16, 4) == 0
    assert e.pending() == (0, 0)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("n", [5, 4099, util.STREAM_SIZE])
def test_incr_mode_is_op_then_add(fresh, n, dt):
    # ExternalOp.Do in Incr mode (execution.go:113-127): CUDADo into a temporary, then an unsafe add into
    # op.Incr. One fused kernel here, the temporary never stored, the arena back where it was.
    e = fresh
    a, b, c = util.normal(31, n, dt), util.normal(32, n, dt), util.normal(33, n, dt)
    ta, tb, tc = e.tensor(a), e.tensor(b), e.tensor(c)
    e.Signal()
    used, l0 = e.arena_stats()["used"], e.launches
    e.BinaryIncr("mul", ta, tb, tc)
    assert e.pending() == (2, 1)
    got = tc.numpy()
    assert e.launches == l0 + 1
    assert e.arena_stats()["used"] == used
    assert_bits_equal(got, oracle.binary("add", c, oracle.binary("mul", a, b)))
    # scalar forms and a unary op
    e.BinaryIncr("sub", ta, 2.5, tc)
    want = oracle.binary("add", got, oracle.binary("sub", a, dt(2.5)))
    assert_bits_equal(tc.numpy(), want)
    e.BinaryIncr("div", 2.0, tb, tc)
    want = oracle.binary("add", want, oracle.binary("div", dt(2.0), b))
    assert_bits_equal(tc.numpy(), want)
    e.UnaryIncr("tanh", ta, tc)
    th = oracle.unary("tanh", a)
    # the op's own 1e-6 is relative to tanh(a), not to a sum that may cancel
    err = np.abs(tc.numpy().astype(np.float64) - oracle.binary("add", want, th))
    assert np.all(err <= (2e-6 if dt == np.float32 else 1e-13) * (np.abs(th) + np.abs(want)))


def test_incr_mode_unfused_engine_gives_the_same_bits():
    from gorgonia_b200 import Engine
    n = 100_003
    a, b, c = util.normal(34, n), util.normal(35, n), util.normal(36, n)
    outs = []
    for defer in (True, False):
        e = Engine(0, 64 << 20, defer=defer)
        ta, tb, tc = e.tensor(a), e.tensor(b), e.tensor(c)
        e.BinaryIncr("pow", e.tensor(np.abs(a) + np.float32(0.1)), tb, tc)
        outs.append(tc.numpy())
        e.Close()
    assert_bits_equal(outs[0], outs[1])

"""Pins the CPU oracle to the golden vectors gorgonia's own tests hold for this path (CPU only).

The fixtures under tests/golden/ were extracted from the Go test files by
tests/golden/extract_goldens.py; each test names the table it checks."""
import numpy as np
import pytest

from oracle import oracle
from tests import golden_util as G


def test_binop_table():
    """binOpTests (op_math_test.go:23-359): values of + - * / in vv, vs, sv and ss forms, f64 and f32."""
    cases = G.load("binop.json")["cases"]
    assert len(cases) >= 30
    n = 0
    for c in cases:
        if c["op"] == "BatchedMatMul":
            a, b = G.arr(c["a"]), G.arr(c["b"])
            got = oracle.batched_matmul(a, b)
            assert got.shape == tuple(c["correct_shape"])
            assert got.reshape(-1).tolist() == c["correct"]["data"]
        else:
            a, b = G.arr(c["a"]), G.arr(c["b"])
            got = oracle.binary(G.BINOPS[c["op"]], a, b)
            want = G.arr(c["correct"])
            assert got.dtype == want.dtype
            assert got.reshape(-1).tolist() == want.reshape(-1).tolist(), c
        n += 1
    assert n == len(cases)


def test_softmax_table():
    """testCasesSoftMaxDo (op_softmax_test.go:13-99): float64 goldens at the 1e-16 level."""
    for c in G.load("softmax_do.json")["cases"]:
        x = np.array(c["input"], np.float64).reshape(c["shape"])
        got = oracle.softmax(x, -1)
        np.testing.assert_allclose(got.reshape(-1), np.array(c["expected"]), rtol=1e-14, atol=0)
        got32 = oracle.softmax(x.astype(np.float32), -1)
        np.testing.assert_allclose(got32.reshape(-1), np.array(c["expected"]), rtol=2e-6, atol=0)


def test_maxpool_asymmetric_padding():
    """TestMaxPool2D_asymmetricPadding (nn_test.go:91-138): pins the south/east origin of explicit padding."""
    d = G.load("maxpool_asym.json")
    for c in d["cases"]:
        x, want = G.arr(c["input"]), G.arr(c["output"])
        got, _ = oracle.maxpool2d(x.astype(np.float32), d["kernel"], d["pad"], d["stride"])
        assert got.shape == want.shape
        assert np.array_equal(got, want.astype(np.float32))


def test_maxpool_basic():
    for c in G.load("maxpool_basic.json")["cases"]:
        got, _ = oracle.maxpool2d(G.arr(c["input"]).astype(np.float32), c["kernel"], c["pad"], c["stride"])
        assert list(got.shape) == c["expected_shape"] and got.reshape(-1).tolist() == c["expected"]


def test_conv_issue233():
    """TestIssue233_F32/_F64 (known_issues_test.go:160-239): Conv2d 3x3 pad 1 on a 5x5 ramp."""
    for c in G.load("conv_issue233.json")["cases"]:
        got = oracle.conv2d(G.arr(c["x"]), G.arr(c["w"]), c["pad"], c["stride"], c["dilation"])
        assert got.reshape(-1).tolist() == c["correct"]


def test_leaky_relu():
    """TestLeakyRelu (nn_test.go:538-588), held there to 1e-6 absolute."""
    for c in G.load("leakyrelu.json")["cases"]:
        x, want = G.arr(c["x"]), G.arr(c["y"])
        got = oracle.leaky_relu(x, c["alpha"])
        np.testing.assert_allclose(got, want, rtol=0, atol=1e-6)


def test_by_indices():
    """TestByIndicesOpDo (op_by_indices_test.go:12-86), axis 0 and axis 1."""
    for c in G.load("byindices.json")["cases"]:
        got = oracle.gather_axis(G.arr(c["input"]), G.arr(c["indices"]), c["axis"])
        assert list(got.shape) == c["expected_shape"] and got.reshape(-1).tolist() == c["expected"]


def test_broadcast_add():
    """broadcastAddTests (operations_broadcast_test.go:24-73): the six vector/matrix forms."""
    for c in G.load("broadcast_add.json")["cases"]:
        div, mod, small_is_a = G.broadcast_div_mod(c)
        a, b = G.arr(c["a"]).reshape(-1), G.arr(c["b"]).reshape(-1)
        full_shape = (c["b"] if small_is_a else c["a"])["shape"]
        a2 = a if small_is_a else a.reshape(full_shape)
        b2 = b.reshape(full_shape) if small_is_a else b
        got = oracle.binary_bcast("add", a2, b2, div, mod, small_is_a)
        assert got.reshape(-1).tolist() == c["ab"]["data"], c["name"]


def test_fixtures_match_the_generator_if_a_checkout_is_given():
    """With GORGONIA_SRC pointing at a gorgonia checkout, the committed fixtures equal a fresh extraction."""
    import json
    import os
    root = os.environ.get("GORGONIA_SRC", "")
    if not root or not os.path.exists(os.path.join(root, "op_math_test.go")):
        pytest.skip("set GORGONIA_SRC to a gorgonia checkout to run this check")
    from tests.golden import extract_goldens as X
    assert X.extract_binop(root) == json.load(open(os.path.join(G.GOLDEN, "binop.json")))
    for name, fn in (("byindices", X.extract_byindices), ("softmax_do", X.extract_softmax),
                     ("maxpool_asym", X.extract_maxpool_asym), ("maxpool_basic", X.extract_maxpool_basic),
                     ("conv_issue233", X.extract_conv), ("leakyrelu", X.extract_leakyrelu),
                     ("broadcast_add", X.extract_broadcast), ("batchnorm", X.extract_batchnorm),
                     ("dropout", X.extract_dropout)):
        assert fn(root) == json.load(open(os.path.join(G.GOLDEN, name + ".json"))), name


# ---- backward ops: known answers derived from the configurations of gorgonia's own tests ---------

def test_oracle_maxpool_bwd_known_answer():
    # nn_test.go:140-193 (TestMaxPool2D): x = 0..23 as (1,2,3,4), 2x2 window, stride 1, cost = Sum(y).
    # x increases along both axes, so every window's maximum is its last element and the gradient is
    # 1 where h >= 1 and w >= 1, 0 elsewhere.
    x = np.arange(24, dtype=np.float32).reshape(1, 2, 3, 4)
    y, mask = oracle.maxpool2d(x, (2, 2), (0, 0), (1, 1))
    dx = oracle.maxpool2d_bwd(np.ones_like(y), mask, x.shape)
    want = np.zeros_like(x)
    want[:, :, 1:, 1:] = 1
    assert np.array_equal(dx, want)


@pytest.mark.parametrize("kernel,pad,stride", [((4, 4), (0, 0), (1, 1)), ((3, 3), (1, 1), (2, 2)),
                                                ((3, 3), (1, 1), (3, 3))])
def test_oracle_col2im_counts_windows(kernel, pad, stride):
    # nn_test.go:13-89 (TestIm2Col): the gradient of Sum(Im2Col(x)) is col2im(ones), which counts the
    # windows that cover each pixel; the count is recomputed here pixel by pixel.
    shape = (2, 1, 28, 28)
    Ho, Wo = oracle.conv_out(28, kernel[0], pad[0], stride[0]), oracle.conv_out(28, kernel[1], pad[1], stride[1])
    ones = np.ones((2, Ho, Wo, kernel[0] * kernel[1]), np.float32)
    got = oracle.col2im(ones, shape, kernel[0], kernel[1], pad, stride)
    want = np.zeros((28, 28), np.float32)
    for ih in range(28):
        for iw in range(28):
            n = 0
            for r in range(kernel[0]):
                for s in range(kernel[1]):
                    a, b = ih + pad[0] - r, iw + pad[1] - s
                    if a >= 0 and b >= 0 and a % stride[0] == 0 and b % stride[1] == 0 and a // stride[0] < Ho \
                            and b // stride[1] < Wo:
                        n += 1
            want[ih, iw] = n
    assert np.array_equal(got, np.broadcast_to(want, shape))


@pytest.mark.parametrize("log", [False, True])
def test_oracle_softmax_bwd_matches_finite_differences(log):
    # no vector for SoftMaxB / LogSoftMaxB exists in gorgonia's tests: check the restated formula
    # against central differences of the oracle's own forward op, in float64
    g = np.random.Generator(np.random.Philox(11))
    x, gr = g.standard_normal((4, 6)), g.standard_normal((4, 6))
    y = oracle.softmax(x, -1, log)
    got = oracle.softmax_bwd(y, gr, -1, log)
    h = 1e-6
    want = np.zeros_like(x)
    for i in range(4):
        for j in range(6):
            xp, xm = x.copy(), x.copy()
            xp[i, j] += h
            xm[i, j] -= h
            want[i, j] = ((oracle.softmax(xp, -1, log) - oracle.softmax(xm, -1, log)) * gr).sum() / (2 * h)
    assert np.abs(got - want).max() < 1e-8


# ---- BatchNormOp: the ten cases of bnAllCases ----------------------------------------------------

def _bn_init(spec, n, dt):
    if spec["kind"] == "ranged":      # RangedFromWithStep (weights.go:56-120): repeated addition in the tensor's type
        out, st, inc = np.empty(n, dt), dt(spec["start"]), dt(spec["step"])
        for i in range(n):
            out[i] = st
            st = dt(st + inc)
        return out
    if spec["kind"] == "ones":
        return np.ones(n, dt)
    if spec["kind"] == "zeroes":
        return np.zeros(n, dt)
    return np.asarray(spec["data"], dtype=dt)


def bn_case_arrays(case):
    dt = np.float32 if case["dtype"] == "float32" else np.float64
    shape = tuple(case["x_shape"])
    n = int(np.prod(shape))
    x = _bn_init(case["x"], n, dt).reshape(shape)
    bshape = (1, shape[1]) + (1,) * (len(shape) - 2)
    scale = _bn_init(case["scale"], shape[1], dt).reshape(bshape)
    bias = _bn_init(case["bias"], shape[1], dt).reshape(bshape)
    fc = _bn_init(case["scale"], n, dt).reshape(shape[0], n // shape[0])
    return dt, x, scale, bias, fc


@pytest.mark.parametrize("case", G.load("batchnorm.json")["cases"], ids=lambda c: c["desc"] + " " + c["dtype"])
def test_oracle_batchnorm_goldens(case):
    # nn_test.go:319-440: one training run from running mean 0 / running variance 1; the test reads the
    # running statistics and ((BatchNorm(x) * scale + bias) as (B, F)) x fcWeight^T
    dt, x, scale, bias, fc = bn_case_arrays(case)
    rm, rv = np.zeros(x.shape[1], dt), np.ones(x.shape[1], dt)
    y, _, _ = oracle.batchnorm(x, rm, rv, training=True, momentum=0.9, eps=1e-5)
    tol = 1e-5 if dt == np.float32 else 1e-9
    assert np.allclose(rm, np.asarray(case["running_mean"], dt), rtol=tol, atol=tol)
    assert np.allclose(rv, np.asarray(case["running_var"], dt), rtol=tol, atol=tol)
    out = ((y * scale).astype(dt) + bias).astype(dt).reshape(x.shape[0], -1) @ fc.T
    want = np.asarray(case["train_result"], dt).reshape(out.shape)
    assert np.allclose(out, want, rtol=10 * tol, atol=10 * tol)


def test_dropout_goldens():
    """TestDropoutAll (op_dropout_test.go:14-68): x = ones(5), the injected generator cycles through `rand`,
    cost = Mean(y), so dcost/dy = 1/5; forward output and input gradient as the reference expects them
    (the gradient divides by the drop probability, and is 0 where the output is 0)."""
    for c in G.load("dropout.json")["cases"]:
        dt = G.DT[c["dtype"]]
        x = np.ones(5, dt)
        y = oracle.dropout(x, c["prob"], uniforms=np.array(c["rand"], dt))
        assert y.tolist() == c["y"], c
        dy = np.array(c["y_grad"], dt)
        dx = oracle.dropout_bwd(dy, y, c["prob"])
        want = np.array(c["x_grad"], dt)
        assert np.allclose(dx, want, rtol=1e-6 if dt == np.float32 else 1e-15, atol=0), (c, dx)


def test_dropout_philox_statistics():
    # the stateless generator: uniform on [0, 1), the kept share matches 1 - p, replays are identical
    x = np.ones(200_000, np.float32)
    y = oracle.dropout(x, 0.3, seed=1234)
    kept = float((y != 0).mean())
    assert abs(kept - 0.7) < 0.005
    assert np.all((y == 0) | (y == np.float32(1) / np.float32(0.7)))
    assert np.array_equal(y, oracle.dropout(x, 0.3, seed=1234))
    assert not np.array_equal(y, oracle.dropout(x, 0.3, seed=1235))
    # an offset continues the same stream
    assert np.array_equal(oracle.dropout(x[:1000], 0.3, seed=1234, offset=5000), y[5000:6000])


def _oldsoftmax_grad(a, g, axis):
    """The gradient of gorgonia's second softmax formulation, oldsoftmax = Exp -> Sum -> broadcast Div
    (op_softmax_test.go:239-282), composed from the primitive differentiation rules in double:
    Div: d(e/s)/de = 1/s, d(e/s)/ds = -e/s^2; Sum: its gradient is repeated along the axis; Exp: de/da = e."""
    a = a.astype(np.float64)
    e = np.exp(a)
    s = e.sum(axis=axis, keepdims=True)
    de = g / s
    ds = -(g * e / (s * s)).sum(axis=axis, keepdims=True)
    return (de + ds) * e


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_softmax_bwd_agrees_with_the_old_softmax_composition(dt):
    # TestOld_NewSoftmax (op_softmax_test.go:284-330) builds both formulations on this input with cost =
    # Sum(softmax): the gradient is zero up to rounding, whichever way it is formed
    a = np.array([0.1, 0.1, 0.3, 0.1, 0.4], dt)
    y = oracle.softmax(a)
    dx = oracle.softmax_bwd(y, np.ones_like(a))
    assert np.abs(dx).max() <= (1e-7 if dt == np.float32 else 1e-16)
    assert np.abs(_oldsoftmax_grad(a, np.ones(5), 0)).max() <= 1e-16
    # with an upstream gradient that does not cancel, on matrices and on a middle axis
    for shape, axis in (((5,), 0), ((7, 10), 1), ((4, 6, 3), 1)):
        x = np.random.Generator(np.random.Philox(5)).standard_normal(shape).astype(dt)
        g = np.random.Generator(np.random.Philox(6)).standard_normal(shape).astype(dt)
        got = oracle.softmax_bwd(oracle.softmax(x, axis), g, axis)
        want = _oldsoftmax_grad(x, g.astype(np.float64), axis)
        assert np.allclose(got, want, rtol=2e-5 if dt == np.float32 else 1e-12, atol=2e-6 if dt == np.float32 else 1e-14)
        # log-softmax = Log(oldsoftmax): one more primitive rule, d log(y) = g / y
        yl = oracle.softmax(x, axis, log=True)
        gotl = oracle.softmax_bwd(yl, g, axis, log=True)
        ysm = np.exp(yl.astype(np.float64))
        wantl = _oldsoftmax_grad(x, g.astype(np.float64) / ysm, axis)
        assert np.allclose(gotl, wantl, rtol=2e-5 if dt == np.float32 else 1e-11, atol=2e-5 if dt == np.float32 else 1e-13)

"""The engine against the golden vectors of gorgonia's own tests (GPU, through the C ABI): what
TestCUDABasicArithmetic does with binOpTests on the reference's GPU path
(op_math_cuda_test.go:39-109), extended to the nn tables."""
import numpy as np
import pytest

from tests import golden_util as G

pytestmark = pytest.mark.gpu


def test_binop_table(fresh):
    e = fresh
    for c in G.load("binop.json")["cases"]:
        a, b, want = G.arr(c["a"]), G.arr(c["b"]), G.arr(c["correct"])
        if c["op"] == "BatchedMatMul":
            out = e.empty(c["correct_shape"], a.dtype)
            e.MatMul(e.tensor(a), e.tensor(b), out)
            assert out.numpy().reshape(-1).tolist() == want.reshape(-1).tolist()
            continue
        op = G.BINOPS[c["op"]]
        if a.ndim and b.ndim:
            ta = e.tensor(a)
            e._binary(op, ta, e.tensor(b), unsafe=True)
            got = ta.numpy()
        elif a.ndim:                     # tensor op scalar
            ta = e.tensor(a)
            e._binary_scalar(op, ta, float(b), leftTensor=True, unsafe=True)
            got = ta.numpy()
        elif b.ndim:                     # scalar op tensor: lands in the tensor's buffer
            tb = e.tensor(b)
            e._binary_scalar(op, tb, float(a), leftTensor=False, unsafe=True)
            got = tb.numpy()
        else:                            # scalar op scalar: two one-element device buffers
            ta = e.tensor(a.reshape(1))
            e._binary(op, ta, e.tensor(b.reshape(1)), unsafe=True)
            got = ta.numpy()
        assert got.dtype == want.dtype
        assert got.reshape(-1).tolist() == want.reshape(-1).tolist(), c


def test_softmax_table(fresh):
    e = fresh
    for c in G.load("softmax_do.json")["cases"]:
        for dt, tol in ((np.float64, 1e-13), (np.float32, 2e-6)):
            x = np.array(c["input"], dt).reshape(c["shape"])
            y = e.empty(x.shape, dt)
            e.SoftMax(e.tensor(x), y)
            np.testing.assert_allclose(y.numpy().reshape(-1), np.array(c["expected"]), rtol=tol, atol=0)


def test_maxpool_tables(fresh):
    e = fresh
    d = G.load("maxpool_asym.json")
    for c in d["cases"]:
        x, want = G.arr(c["input"]), G.arr(c["output"])
        y = e.empty(want.shape, x.dtype)
        e.MaxPool2D(e.tensor(x), y, d["kernel"], d["pad"], d["stride"])
        assert np.array_equal(y.numpy(), want)
    for c in G.load("maxpool_basic.json")["cases"]:
        x = G.arr(c["input"])
        y = e.empty(c["expected_shape"], x.dtype)
        e.MaxPool2D(e.tensor(x), y, c["kernel"], c["pad"], c["stride"])
        assert y.numpy().reshape(-1).tolist() == c["expected"]


def test_conv_issue233(fresh):
    e = fresh
    for c in G.load("conv_issue233.json")["cases"]:
        x, w = G.arr(c["x"]), G.arr(c["w"])
        y = e.empty((1, 1, 5, 5), x.dtype)
        e.Conv2d(e.tensor(x), e.tensor(w), y, c["pad"], c["stride"], c["dilation"])
        assert y.numpy().reshape(-1).tolist() == c["correct"]


def test_leaky_relu(fresh):
    e = fresh
    for c in G.load("leakyrelu.json")["cases"]:
        x, want = G.arr(c["x"]), G.arr(c["y"])
        tx = e.tensor(x.reshape(-1))
        n, alpha = x.size, c["alpha"]
        p, m, r = e.empty(n, x.dtype), e.empty(n, x.dtype), e.empty(n, x.dtype)
        e.GteScalar(tx, 0.0, reuse=p)       # the six instructions of nn.go:104-130
        e.LtScalar(tx, 0.0, reuse=m)
        e.Mul(tx, p, reuse=p)
        e.Mul(tx, m, reuse=m)
        e.MulScalar(m, alpha if x.dtype == np.float64 else float(np.float32(alpha)), unsafe=True)
        e.Add(p, m, reuse=r)
        np.testing.assert_allclose(r.numpy().reshape(x.shape), want, rtol=0, atol=1e-6)


def test_by_indices(fresh):
    e = fresh
    for c in G.load("byindices.json")["cases"]:
        x, idx = G.arr(c["input"]), G.arr(c["indices"])
        y = e.empty(c["expected_shape"], x.dtype)
        e.ByIndices(e.tensor(x), e.tensor(idx), y, axis=c["axis"])
        assert y.numpy().reshape(-1).tolist() == c["expected"]


def test_broadcast_add(fresh):
    e = fresh
    for c in G.load("broadcast_add.json")["cases"]:
        div, mod, small_is_a = G.broadcast_div_mod(c)
        a, b = G.arr(c["a"]), G.arr(c["b"])
        out = e.empty(c["ab"]["shape"], a.dtype)
        e.BroadcastBinary("add", e.tensor(a), e.tensor(b), div, mod, bcast_is_a=small_is_a, reuse=out)
        assert out.numpy().reshape(-1).tolist() == c["ab"]["data"], c["name"]

"""Backward ops of the training variant: maxPoolDiff, col2im, softmaxDiff, Incr-mode MatMul.

The integer-indexed ops (maxpool gradient, col2im) must equal the oracle bit for bit, also where
windows overlap and several additions land on one element; the floating-point ones carry the
tolerance written in each test."""
import numpy as np
import pytest

from tests import util
from oracle import oracle
from tests.util import assert_bits_equal, assert_gemm_close

pytestmark = pytest.mark.gpu

POOL_BWD_CASES = [
    # shape, kernel, pad, stride
    ((1, 2, 3, 4), (2, 2), (0, 0), (1, 1)),          # TestMaxPool2D's configuration (nn_test.go:140-193)
    ((2, 3, 28, 28), (2, 2), (0, 0), (2, 2)),        # the pools of LeNet / tiny-YOLO
    ((2, 3, 13, 13), (2, 2), (1, 0, 1, 0), (1, 1)),  # tiny-YOLO's last pool: explicit padding, overlapping windows
    ((3, 2, 9, 11), (3, 3), (1, 1), (2, 2)),         # overlapping 3x3 / 2
    ((2, 2, 8, 8), (3, 2), (1, 0), (1, 2)),
    ((1, 1, 7, 7), (2, 2), (0, 0), (2, 2)),          # odd planes: a row and a column belong to no window
    ((2, 4, 6, 6), (5, 5), (2, 2), (1, 1)),          # every element sits in up to 25 windows
]


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("shape,kernel,pad,stride", POOL_BWD_CASES)
def test_maxpool_bwd_bit_exact(fresh, shape, kernel, pad, stride, dt):
    e = fresh
    x = util.normal(61, shape, dt)
    # ties on purpose: quantise so that several window elements share the maximum
    x = (np.round(x * 2) / 2).astype(dt)
    want_y, want_mask = oracle.maxpool2d(x.astype(np.float32), kernel, pad, stride)
    y = e.empty(want_y.shape, dt)
    mask = e.empty(want_y.shape, np.int64)
    e.MaxPool2D(e.tensor(x), y, kernel, pad, stride, mask=mask)
    assert np.array_equal(mask.numpy(), want_mask)
    dy = util.normal(62, want_y.shape, dt)
    dx = e.empty(shape, dt)
    e.MaxPool2DDiff(e.tensor(dy), mask, dx, kernel, pad, stride)
    assert_bits_equal(dx.numpy(), oracle.maxpool2d_bwd(dy, want_mask, shape))


def test_maxpool_bwd_known_answer(fresh):
    # nn_test.go:140-193: x = 0..23 as (1,2,3,4), 2x2 / stride 1, cost = Sum(y). Every window's
    # maximum is its last element, so the gradient is 1 where h >= 1 and w >= 1 and 0 elsewhere.
    e = fresh
    x = np.arange(24, dtype=np.float32).reshape(1, 2, 3, 4)
    y, mask = e.empty((1, 2, 2, 3)), e.empty((1, 2, 2, 3), np.int64)
    e.MaxPool2D(e.tensor(x), y, (2, 2), (0, 0), (1, 1), mask=mask)
    dx = e.empty(x.shape)
    e.MaxPool2DDiff(e.tensor(np.ones((1, 2, 2, 3), np.float32)), mask, dx, (2, 2), (0, 0), (1, 1))
    want = np.zeros_like(x)
    want[:, :, 1:, 1:] = 1
    assert_bits_equal(dx.numpy(), want)


COL2IM_CASES = [
    # image shape, kernel, pad, stride, dilation
    ((2, 1, 28, 28), (4, 4), (0, 0), (1, 1), (1, 1)),   # im2colTests (nn_test.go:13-23)
    ((2, 1, 28, 28), (3, 3), (1, 1), (2, 2), (1, 1)),
    ((2, 1, 28, 28), (3, 3), (1, 1), (3, 3), (1, 1)),
    ((2, 3, 9, 8), (3, 3), (1, 1), (1, 1), (1, 1)),
    ((1, 4, 20, 20), (3, 3), (2, 2), (1, 1), (2, 2)),   # dilation
    ((2, 5, 17, 19), (3, 5), (2, 1), (2, 3), (1, 1)),   # odd everything
    ((3, 2, 6, 6), (1, 1), (0, 0), (1, 1), (1, 1)),     # 1x1: a plain transposition
    # 3 x 3, unit stride, C * 9 a multiple of 4: float32 takes the bulk-copy ring kernel
    ((5, 32, 14, 14), (3, 3), (1, 1), (1, 1), (1, 1)),  # LeNet's conv1
    ((700, 4, 10, 12), (3, 3), (1, 1), (1, 1), (1, 1)), # more images than resident blocks: the ring runs across images
    ((3, 8, 9, 11), (3, 3), (0, 0), (1, 1), (1, 1)),    # no padding: fewer col rows than image rows
    ((3, 8, 7, 6), (3, 3), (2, 2), (1, 1), (1, 1)),     # full padding: more col rows than image rows
    ((2, 4, 2, 4), (3, 3), (1, 1), (1, 1), (1, 1)),     # an image shorter than the window
]


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("shape,kernel,pad,stride,dil", COL2IM_CASES)
def test_col2im_bit_exact(fresh, shape, kernel, pad, stride, dil, dt):
    e = fresh
    B, Cc, H, W = shape
    Ho = oracle.conv_out(H, kernel[0], pad[0], stride[0], dil[0])
    Wo = oracle.conv_out(W, kernel[1], pad[1], stride[1], dil[1])
    col = util.normal(63, (B, Ho, Wo, Cc * kernel[0] * kernel[1]), dt)
    im = e.empty(shape, dt)
    e.Col2Im(e.tensor(col), im, kernel, pad, stride, dil)
    assert_bits_equal(im.numpy(), oracle.col2im(col, shape, kernel[0], kernel[1], pad, stride, dil))


def test_col2im_is_the_adjoint_of_im2col(fresh):
    # <im2col(x), c> == <x, col2im(c)>, and col2im(ones) counts the windows that cover each pixel
    e = fresh
    shape, kernel, pad, stride = (2, 3, 12, 10), (3, 3), (1, 1), (2, 2)
    x = util.normal(64, shape, np.float64)
    Ho, Wo = oracle.conv_out(12, 3, 1, 2), oracle.conv_out(10, 3, 1, 2)
    c = util.normal(65, (2, Ho, Wo, 27), np.float64)
    col, im = e.empty(c.shape, np.float64), e.empty(shape, np.float64)
    e.Im2Col(e.tensor(x), col, kernel, pad, stride)
    e.Col2Im(e.tensor(c), im, kernel, pad, stride)
    lhs, rhs = float((col.numpy() * c).sum()), float((x * im.numpy()).sum())
    assert abs(lhs - rhs) <= 1e-12 * max(abs(lhs), 1.0)
    ones = e.empty(shape, np.float64)
    e.Col2Im(e.tensor(np.ones_like(c)), ones, kernel, pad, stride)
    count = np.zeros(shape[2:])
    for oh in range(Ho):
        for ow in range(Wo):
            for r in range(3):
                for s in range(3):
                    ih, iw = oh * 2 - 1 + r, ow * 2 - 1 + s
                    if 0 <= ih < 12 and 0 <= iw < 10:
                        count[ih, iw] += 1
    assert np.array_equal(ones.numpy(), np.broadcast_to(count, shape))


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("log", [False, True])
@pytest.mark.parametrize("shape,axis", [((256, 10), 1), ((8192, 10), -1), ((7, 3), 1), ((33, 1000), 1),
                                        ((5, 6, 7), 1), ((4, 5000), 1), ((10, 1), 0)])
def test_softmax_bwd(fresh, shape, axis, log, dt):
    # tolerance: 1e-6 (float32) / 1e-13 (float64) of max(|r|, the largest |grad| of the tensor): the
    # difference g - sum(g*y) cancels, so an element-wise relative bound would be ill-posed
    e = fresh
    x = util.normal(66, shape, dt)
    y = oracle.softmax(x, axis, log)
    g = util.normal(67, shape, dt)
    want = oracle.softmax_bwd(y, g, axis, log)
    dx = e.empty(shape, dt)
    e.SoftMaxDiff(e.tensor(y), e.tensor(g), dx, axis, log)
    got = dx.numpy()
    rel = 1e-6 if dt == np.float32 else 1e-13
    lim = rel * np.maximum(np.abs(want.astype(np.float64)), float(np.abs(g).max()))
    assert (np.abs(got.astype(np.float64) - want.astype(np.float64)) <= lim).all()
    if not log:   # sum_i y_i = 1, so the derivative sums to zero along the axis
        assert np.abs(got.astype(np.float64).sum(axis)).max() <= (1e-5 if dt == np.float32 else 1e-12) * np.abs(g).max()


@pytest.mark.parametrize("shape", [(300, 200, 512), (128, 128, 64), (257, 130, 96), (33, 7, 20)])
def test_matmul_incr_equals_product_then_add(fresh, shape):
    # Incr mode (execution.go:115-126): the product is rounded to float32, then added to what the
    # output holds; one call must equal MatMul into a temporary followed by Add, bit for bit
    e = fresh
    M, N, K = shape
    a, b = util.normal(68, (M, K), scale=0.05), util.normal(69, (K, N), scale=0.05)
    c0 = util.normal(70, (M, N))
    ta, tb = e.tensor(a), e.tensor(b)
    c = e.tensor(c0)
    e.MatMul(ta, tb, c, incr=True)
    tmp, ref = e.empty((M, N)), e.tensor(c0)
    e.MatMul(ta, tb, tmp)
    e.Add(ref, tmp, unsafe=True)
    assert_bits_equal(c.numpy(), ref.numpy())
    assert_gemm_close(c.numpy(), c0.astype(np.float64) + oracle.gemm(a, b).astype(np.float64), 1e-5)


def test_matmul_incr_float64(fresh):
    e = fresh
    a, b = util.normal(71, (40, 30), np.float64), util.normal(72, (30, 20), np.float64)
    c0 = util.normal(73, (40, 20), np.float64)
    c = e.tensor(c0)
    e.MatMul(e.tensor(a), e.tensor(b), c, incr=True)
    assert np.abs(c.numpy() - (c0 + a @ b)).max() <= 1e-12


# ---- BatchNormOp (the cuDNN-free forward) -----------------------------------------------------

from tests import golden_util as G  # noqa: E402
from tests.test_oracle_golden import bn_case_arrays  # noqa: E402


@pytest.mark.parametrize("case", G.load("batchnorm.json")["cases"], ids=lambda c: c["desc"] + " " + c["dtype"])
def test_batchnorm_goldens(fresh, case):
    # nn_test.go:319-440 / nn_amd64_test.go: one training run from running mean 0, running variance 1
    e = fresh
    dt, x, scale, bias, fc = bn_case_arrays(case)
    Cc = x.shape[1]
    rm, rv = e.tensor(np.zeros(Cc, dt)), e.tensor(np.ones(Cc, dt))
    sm, sv = e.empty((Cc,), dt), e.empty((Cc,), dt)
    y = e.empty(x.shape, dt)
    e.BatchNorm(e.tensor(x), y, rm, rv, sm, sv, training=True, momentum=0.9, epsilon=1e-5)
    tol = 1e-5 if dt == np.float32 else 1e-9
    assert np.allclose(rm.numpy(), np.asarray(case["running_mean"], dt), rtol=tol, atol=tol)
    assert np.allclose(rv.numpy(), np.asarray(case["running_var"], dt), rtol=tol, atol=tol)
    out = ((y.numpy() * scale).astype(dt) + bias).astype(dt).reshape(x.shape[0], -1) @ fc.T
    assert np.allclose(out, np.asarray(case["train_result"], dt).reshape(out.shape), rtol=10 * tol, atol=10 * tol)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("shape", [(64, 10), (300, 625), (8, 3, 5, 7), (16, 32, 14, 14), (2, 4, 64, 64), (70, 1, 3, 3)])
def test_batchnorm_training_and_inference(fresh, shape, dt):
    # statistics: 2e-6 (float32) / 1e-12 (float64) of their magnitude: the reference sums sequentially
    # in the tensor's type, the device in double; output: the pointwise tolerance on the scale of the
    # largest |y|; inference (given statistics, no sums) is bit-exact
    e = fresh
    x = (util.normal(81, shape, dt) * dt(1.7) + dt(0.3)).astype(dt)
    Cc = shape[1]
    rm0, rv0 = util.normal(82, Cc, dt), (np.abs(util.normal(83, Cc, dt)) + dt(0.5)).astype(dt)
    rm_o, rv_o = rm0.copy(), rv0.copy()
    want, sm_o, sv_o = oracle.batchnorm(x, rm_o, rv_o, training=True, momentum=0.9, eps=1e-5)
    rm, rv = e.tensor(rm0), e.tensor(rv0)
    sm, sv, y = e.empty((Cc,), dt), e.empty((Cc,), dt), e.empty(shape, dt)
    tx = e.tensor(x)
    e.BatchNorm(tx, y, rm, rv, sm, sv, training=True, momentum=0.9, epsilon=1e-5)
    st = 2e-6 if dt == np.float32 else 1e-12
    for got, ref in ((sm.numpy(), sm_o), (sv.numpy(), sv_o), (rm.numpy(), rm_o), (rv.numpy(), rv_o)):
        assert np.abs(got.astype(np.float64) - ref).max() <= st * max(1.0, np.abs(ref).max()) * (10 if ref is sv_o else 1)
    lim = (1e-5 if dt == np.float32 else 1e-11) * max(1.0, float(np.abs(want).max()))
    assert np.abs(y.numpy().astype(np.float64) - want).max() <= lim
    # inference with the statistics the oracle ended with: no sums involved, bit-exact
    rm2, rv2 = e.tensor(rm_o), e.tensor(rv_o)
    e.BatchNorm(tx, y, rm2, rv2, training=False, momentum=0.9, epsilon=1e-5)
    want_inf, _, _ = oracle.batchnorm(x, rm_o.copy(), rv_o.copy(), training=False, momentum=0.9, eps=1e-5)
    assert_bits_equal(y.numpy(), want_inf)
    assert_bits_equal(rm2.numpy(), rm_o)       # untouched


@pytest.mark.parametrize("training", [True, False])
@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("shape", [(64, 10), (300, 33), (8, 3, 5, 7), (16, 32, 14, 14), (70, 1, 3, 3)])
def test_batchnorm_bwd(fresh, shape, dt, training):
    # tolerance: 1e-5 (float32) / 1e-11 (float64) of the largest |dx|: sums in double on the device,
    # sequential in the tensor's type in the reference; inference mode is a product per element
    e = fresh
    x = (util.normal(84, shape, dt) * dt(1.3) + dt(0.2)).astype(dt)
    dy = util.normal(85, shape, dt)
    Cc = shape[1]
    rm, rv = np.zeros(Cc, dt), np.ones(Cc, dt)
    _, sm, sv = oracle.batchnorm(x, rm, rv, training=True)
    want = oracle.batchnorm_bwd(x, dy, rv, sm, sv, training=training)
    dx = e.empty(shape, dt)
    e.BatchNormDiff(e.tensor(x), e.tensor(dy), dx, e.tensor(rv), e.tensor(sm), e.tensor(sv), training=training)
    if not training:
        assert_bits_equal(dx.numpy(), want)
    else:
        lim = (1e-5 if dt == np.float32 else 1e-11) * max(1.0, float(np.abs(want).max()))
        assert np.abs(dx.numpy().astype(np.float64) - want).max() <= lim


def test_dropout_goldens_on_the_device(fresh):
    # TestDropoutAll (op_dropout_test.go:14-68) with its injected generator as a device array
    from tests import golden_util as G
    e = fresh
    for c in G.load("dropout.json")["cases"]:
        dt = G.DT[c["dtype"]]
        tx, tr = e.tensor(np.ones(5, dt)), e.tensor(np.array(c["rand"], dt))
        y, dx = e.empty(5, dt), e.empty(5, dt)
        e.Dropout(tx, y, c["prob"], uniforms=tr)
        assert y.numpy().tolist() == c["y"], c
        e.DropoutDiff(e.tensor(np.array(c["y_grad"], dt)), y, dx, c["prob"])
        assert np.allclose(dx.numpy(), np.array(c["x_grad"], dt), rtol=1e-6 if dt == np.float32 else 1e-15, atol=0)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_dropout_stateless_generator_matches_the_oracle(fresh, dt):
    e = fresh
    n = (1 << 20) + 3
    x = util.normal(80, n, dt)
    tx, y, dx = e.tensor(x), e.empty(n, dt), e.empty(n, dt)
    e.Dropout(tx, y, 0.25, seed=0x1234567890ABCDEF, offset=7)
    want = oracle.dropout(x, 0.25, seed=0x1234567890ABCDEF, offset=7)
    assert_bits_equal(y.numpy(), want)
    assert abs(float((want != 0).mean()) - 0.75) < 0.005
    dy = util.normal(81, n, dt)
    e.DropoutDiff(e.tensor(dy), y, dx, 0.25)
    assert_bits_equal(dx.numpy(), oracle.dropout_bwd(dy, want, 0.25))
    # probability 0 hands the input through; a recorded tape replays the same draw
    e.Dropout(tx, y, 0.0)
    assert_bits_equal(y.numpy(), x)
    e.Signal()
    e.tape_begin()
    e.Dropout(tx, y, 0.5, seed=99)
    t = e.tape_end()
    e.tape_launch(t)
    first = y.numpy()
    e.tape_launch(t)
    assert_bits_equal(y.numpy(), first)
    assert_bits_equal(first, oracle.dropout(x, 0.5, seed=99))
    e.tape_destroy(t)

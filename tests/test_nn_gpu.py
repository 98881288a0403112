"""Parity of softmax, reductions, argmax, conv, im2col, max-pool, transpose and gather against the
CPU oracle (GPU tests). Index-valued results (argmax, pool masks, gathers, transposes) are
bit-exact; softmax is held to the pointwise tolerance, sums and convolutions to the GEMM one."""
import numpy as np
import pytest

from oracle import oracle
from tests import util
from tests.util import assert_bits_equal, assert_gemm_close, assert_pointwise_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("shape,axis", [((1, 1), 1), ((256, 10), 1), ((8192, 10), -1), ((7, 3), 1), ((33, 100), 1),
                                        ((5, 1000), 1), ((3, 2048), 1), ((2, 5000), 1), ((10,), 0), ((6, 5, 4), 1),
                                        ((64, 10, 13, 13), 1), ((300, 7), 0)])
@pytest.mark.parametrize("log", [False, True])
def test_softmax(fresh, shape, axis, log, dt):
    e = fresh
    x = util.normal(51, shape, dt, 2.0)
    y = e.empty(shape, dt)
    e.SoftMax(e.tensor(x), y, axis, log)
    want = oracle.softmax(x, axis, log)
    eps = 2e-6 if dt == np.float32 else 1e-13   # the sum of `len` terms carries log2(len) roundings
    if log:
        # log-softmax is a difference of O(1) quantities: its error is absolute, not relative to
        # a result that may sit arbitrarily close to zero
        err = np.abs(y.numpy().astype(np.float64) - want)
        assert np.all(err <= eps * np.maximum(1.0, np.abs(want)))
    else:
        assert_pointwise_close(y.numpy(), want, eps)


def test_softmax_extremes(fresh):
    e = fresh
    x = np.array([[1000.0, 1000.0, -1000.0], [-1e30, 0.0, 1e30], [0.0, 0.0, 0.0]], dtype=np.float32)
    y = e.empty(x.shape)
    e.SoftMax(e.tensor(x), y)
    assert_pointwise_close(y.numpy(), oracle.softmax(x))


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("shape,axis", [((1, 1), 0), ((256, 10), 1), ((256, 10), 0), ((33, 1000), 1), ((4, 5000), 1),
                                        ((6, 5, 4), 1), ((6, 5, 4), 0), ((2, 3, 4, 5), 2), ((100000,), 0)])
def test_reduce_axis(fresh, shape, axis, dt):
    e = fresh
    x = util.normal(61, shape, dt)
    out_shape = shape[:axis] + shape[axis + 1:]
    for kind in ("sum", "max"):
        y = e.empty(out_shape if out_shape else (1,), dt)
        e.Reduce(kind, e.tensor(x), y, axis)
        want = oracle.reduce(kind, x, axis)
        got = y.numpy().reshape(want.shape)
        if kind == "max":
            assert_bits_equal(got, want)
        else:
            scale = np.abs(x).sum(axis=axis)   # a sum is judged against the magnitude it summed
            assert np.all(np.abs(got.astype(np.float64) - want) <= (1e-6 if dt == np.float32 else 1e-14) * scale + 0)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("n", [1, 31, 1024, 1025, 100_003, 1 << 22])
def test_reduce_all(fresh, n, dt):
    e = fresh
    x = util.normal(71, n, dt)
    tx, y = e.tensor(x), e.empty(1, dt)
    for _ in range(2):                      # twice: the ticket in scratch must re-arm itself
        e.ReduceAll("sum", tx, y)
        want = np.sum(x.astype(np.float64))
        assert abs(float(y.numpy()[0]) - want) <= (1e-6 if dt == np.float32 else 1e-14) * np.abs(x).sum()
        e.ReduceAll("max", tx, y)
        assert y.numpy()[0] == x.max()


def test_argmax_bit_exact(fresh):
    e = fresh
    x = util.normal(81, (4096, 10))
    x[5] = 1.0                              # ties: the first maximum wins
    x[6, 3] = x[6, 7] = 9.0
    y = e.empty((4096,), np.int64)
    e.Argmax(e.tensor(x), y, 1)
    assert np.array_equal(y.numpy(), oracle.argmax(x, 1))
    assert y.numpy()[5] == 0 and y.numpy()[6] == 3
    x3 = util.normal(82, (7, 9, 11))
    y3 = e.empty((7, 11), np.int64)
    e.Argmax(e.tensor(x3), y3, 1)
    assert np.array_equal(y3.numpy(), oracle.argmax(x3, 1))


CONV_CASES = [
    # B, C, H, W, K, kh, kw, pad, stride, dil
    (2, 1, 28, 28, 32, 3, 3, (1, 1), (1, 1), (1, 1)),      # LeNet conv0 shape
    (3, 32, 14, 14, 64, 3, 3, (1, 1), (1, 1), (1, 1)),     # LeNet conv1 shape
    (2, 64, 7, 7, 128, 3, 3, (1, 1), (1, 1), (1, 1)),      # LeNet conv2 shape
    (1, 3, 52, 52, 16, 3, 3, (1, 1), (1, 1), (1, 1)),      # YOLO first-layer shape, small image
    (2, 8, 13, 13, 125, 1, 1, (0, 0), (1, 1), (1, 1)),     # YOLO head: 1x1
    (2, 5, 17, 19, 7, 3, 5, (2, 1), (2, 3), (1, 1)),       # odd everything
    (1, 4, 20, 20, 6, 3, 3, (2, 2), (1, 1), (2, 2)),       # dilation
    (1, 2, 5, 5, 3, 3, 3, (0, 0), (1, 1), (1, 1)),         # tiny: CUDA-core path
    (1, 2, 20, 20, 16, 6, 6, (2, 2), (1, 1), (1, 1)),      # 36 taps per channel: the general gather path
    (70, 3, 12, 12, 20, 3, 3, (1, 1), (1, 1), (1, 1)),     # more images than one scratch chunk holds? (small)
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv2d(fresh, case):
    e = fresh
    B, Cc, H, W, K, kh, kw, pad, stride, dil = case
    x = util.uniform(91, (B, Cc, H, W))
    w = util.normal(92, (K, Cc, kh, kw), scale=float(np.sqrt(2.0 / (Cc * kh * kw))))
    want = oracle.conv2d(x, w, pad, stride, dil)
    y = e.empty(want.shape)
    e.Conv2d(e.tensor(x), e.tensor(w), y, pad, stride, dil)
    assert_gemm_close(y.numpy(), want, 1e-5)
    # fused bias + leaky relu equals oracle conv -> add -> LeakyRelu
    bias = util.normal(93, K, scale=0.1)
    e.Conv2d(e.tensor(x), e.tensor(w), y, pad, stride, dil, bias=e.tensor(bias), act="leaky", alpha=0.1)
    want2 = oracle.leaky_relu((want + bias[None, :, None, None]).astype(np.float32), 0.1)
    assert_gemm_close(y.numpy(), want2, 1e-5)


# inputs of 128 KB or more with C a multiple of 32 and more than one tap: the col operand is built
# by the TMA unit
CONV_TMA_CASES = [
    (8, 32, 20, 20, 64, 3, 3, (1, 1), (1, 1), (1, 1)),
    (4, 32, 40, 36, 32, 3, 3, (1, 1), (1, 1), (1, 1)),     # image rows that are not a multiple of anything
    (5, 64, 12, 12, 130, 3, 3, (1, 1), (1, 1), (1, 1)),    # two column tiles, the second ragged
    (3, 64, 17, 19, 40, 3, 5, (2, 1), (2, 3), (1, 1)),     # odd kernel, pads and strides differ per axis
    (2, 32, 24, 24, 24, 3, 3, (2, 2), (1, 1), (2, 2)),     # dilation
    (4, 64, 26, 26, 125, 1, 2, (0, 1), (1, 1), (1, 1)),    # two taps in a row
    (2, 32, 36, 36, 16, 3, 3, (0, 0), (1, 1), (1, 1)),     # no padding
    (4, 32, 16, 18, 8, 3, 3, (3, 1), (1, 1), (1, 1)),      # padding wider than the kernel reach
    (3, 96, 13, 13, 33, 3, 3, (1, 1), (1, 1), (1, 1)),     # 27 k-blocks: more than one accumulation chain
    (300, 32, 7, 7, 20, 3, 3, (1, 1), (1, 1), (1, 1)),     # tiles that span several images
]


# stride 1, C = 16 / 32 / 64, output planes that 16 x 16 tiles cover well: every tap reads an input
# window held in shared memory
CONV_WIN_CASES = [
    (4, 16, 48, 48, 32, 3, 3, (1, 1), (1, 1), (1, 1)),     # 16-channel rows (tiny-YOLO conv1 shape)
    (3, 32, 30, 45, 64, 3, 3, (1, 1), (1, 1), (1, 1)),     # ragged tiles on both axes
    (2, 64, 32, 32, 70, 3, 3, (1, 1), (1, 1), (1, 1)),     # two channel blocks, two column tiles
    (5, 64, 14, 14, 130, 3, 3, (1, 1), (1, 1), (1, 1)),    # LeNet-sized planes: one tile per image
    (4, 16, 32, 32, 24, 3, 3, (2, 2), (1, 1), (2, 2)),     # dilation
    (4, 16, 28, 28, 16, 5, 5, (2, 2), (1, 1), (1, 1)),     # 25 taps: two accumulation chains
    (2, 32, 46, 31, 40, 1, 3, (0, 1), (1, 1), (1, 1)),     # one row of taps
    (2, 32, 32, 32, 8, 3, 3, (0, 0), (1, 1), (1, 1)),      # no padding
    (2, 32, 29, 29, 8, 2, 2, (1, 1), (1, 1), (1, 1)),      # even kernel
]


@pytest.mark.parametrize("gather", [False, True])
@pytest.mark.parametrize("case", CONV_TMA_CASES + CONV_WIN_CASES)
def test_conv2d_tensor_core_col_paths(case, gather):
    from gorgonia_b200 import Engine, _lib
    B, Cc, H, W, K, kh, kw, pad, stride, dil = case
    e = Engine(device=0, arena_bytes=256 << 20, conv_gather=gather)
    try:
        x = util.uniform(94, (B, Cc, H, W)) - np.float32(0.5)
        w = util.normal(95, (K, Cc, kh, kw), scale=float(np.sqrt(2.0 / (Cc * kh * kw))))
        want = oracle.conv2d(x, w, pad, stride, dil)
        tx, tw = e.tensor(x), e.tensor(w)
        path = e.conv2d_path(tx, tw, pad, stride, dil)
        if gather:
            assert path == _lib.CONV_TC_GATHER
        elif case in CONV_WIN_CASES:
            assert path == _lib.CONV_TC_WINDOW
        else:
            assert path in (_lib.CONV_TC_TMA, _lib.CONV_TC_WINDOW)
        y = e.empty(want.shape)
        e.Conv2d(tx, tw, y, pad, stride, dil)
        assert_gemm_close(y.numpy(), want, 1e-5)
        bias = util.normal(96, K, scale=0.1)
        e.Conv2d(tx, tw, y, pad, stride, dil, bias=e.tensor(bias), act="rectify")
        t = (want + bias[None, :, None, None]).astype(np.float32)
        assert_gemm_close(y.numpy(), t * (t >= 0), 1e-5)
        e.Signal()
    finally:
        e.Close()


CONV_POOL_CASES = [
    # B, C, H, W, K, kh, kw, pad, pool, pool_stride
    (3, 1, 28, 28, 32, 3, 3, (1, 1), (2, 2), (2, 2)),      # first-layer kernel, pooled
    (2, 3, 36, 40, 16, 3, 3, (1, 1), (2, 2), (2, 2)),      # first-layer kernel, 3 channels, 16 filters
    (2, 2, 20, 24, 21, 3, 3, (1, 1), (2, 2), (2, 2)),      # ragged filter count
    (4, 32, 30, 44, 64, 3, 3, (1, 1), (2, 2), (2, 2)),     # window kernel, pooled, ragged tiles
    (4, 16, 48, 48, 40, 3, 3, (1, 1), (2, 2), (2, 2)),     # window kernel, 16-channel rows, two column tiles
    (5, 64, 14, 14, 20, 3, 3, (1, 1), (2, 2), (2, 2)),     # window kernel, one tile per image
    (2, 32, 15, 15, 8, 3, 3, (1, 1), (2, 2), (2, 2)),      # odd planes: the two operations in sequence
    (2, 8, 12, 12, 6, 3, 3, (1, 1), (3, 3), (2, 2)),       # another window: the two operations in sequence
    (3, 64, 7, 7, 16, 3, 3, (1, 1), (2, 2), (2, 2)),       # LeNet conv2: odd planes
]


@pytest.mark.parametrize("act", [None, "rectify", "leaky"])
@pytest.mark.parametrize("case", CONV_POOL_CASES)
def test_conv2d_maxpool_equals_the_two_calls(fresh, case, act):
    e = fresh
    B, Cc, H, W, K, kh, kw, pad, pool, ps = case
    x = util.uniform(97, (B, Cc, H, W)) - np.float32(0.5)
    w = util.normal(98, (K, Cc, kh, kw), scale=float(np.sqrt(2.0 / (Cc * kh * kw))))
    bias = util.normal(99, K, scale=0.1)
    tx, tw, tb = e.tensor(x), e.tensor(w), e.tensor(bias)
    Ho, Wo = H + 2 * pad[0] - (kh - 1), W + 2 * pad[1] - (kw - 1)
    conv = e.empty((B, K, Ho, Wo))
    Hq, Wq = (Ho - pool[0]) // ps[0] + 1, (Wo - pool[1]) // ps[1] + 1
    two, one = e.empty((B, K, Hq, Wq)), e.empty((B, K, Hq, Wq))
    e.Conv2d(tx, tw, conv, pad, bias=tb, act=act, alpha=0.1)
    e.MaxPool2D(conv, two, pool, (0, 0), ps)
    e.Conv2dMaxPool(tx, tw, one, pad, bias=tb, act=act, alpha=0.1, pool=pool, pool_stride=ps)
    assert_bits_equal(one.numpy(), two.numpy())
    assert_bits_equal(one.numpy(), oracle.maxpool2d(conv.numpy(), pool, (0, 0), ps)[0])


def test_conv2d_maxpool_special_values(fresh):
    # an all-NaN / -Inf window yields -MaxFloat32, as maxPoolOp.do does
    e = fresh
    x = np.zeros((1, 1, 4, 4), np.float32)
    x[0, 0, :2, :2] = np.nan
    x[0, 0, :2, 2:] = -np.inf
    w = np.zeros((1, 1, 3, 3), np.float32)
    w[0, 0, 1, 1] = 1.0                                    # identity filter
    conv, two, one = e.empty((1, 1, 4, 4)), e.empty((1, 1, 2, 2)), e.empty((1, 1, 2, 2))
    tx, tw = e.tensor(x), e.tensor(w)
    e.Conv2d(tx, tw, conv, (1, 1))
    e.MaxPool2D(conv, two, (2, 2), (0, 0), (2, 2))
    e.Conv2dMaxPool(tx, tw, one, (1, 1))
    assert_bits_equal(one.numpy(), two.numpy())


def test_conv2d_chain_equals_the_unchained_calls(fresh):
    # three links: first-layer kernel + pool -> window kernel + pool -> im2col-TMA kernel; the tensors
    # between them exist only in the NHWC TF32-split form. Bit-equal to Conv2dMaxPool / Conv2d.
    from gorgonia_b200 import _lib
    e = fresh
    B = 16
    x = util.uniform(101, (B, 3, 32, 32)) - np.float32(0.5)
    w0 = util.normal(102, (32, 3, 3, 3), scale=0.3)
    w1 = util.normal(103, (64, 32, 3, 3), scale=0.1)
    w2 = util.normal(104, (40, 64, 3, 3), scale=0.08)
    b0, b1, b2 = util.normal(105, 32, scale=0.1), util.normal(106, 64, scale=0.1), util.normal(107, 40, scale=0.1)
    tx, tw0, tw1, tw2 = e.tensor(x), e.tensor(w0), e.tensor(w1), e.tensor(w2)
    tb0, tb1, tb2 = e.tensor(b0), e.tensor(b1), e.tensor(b2)
    # unchained
    p0, p1, y2 = e.empty((B, 32, 16, 16)), e.empty((B, 64, 8, 8)), e.empty((B, 40, 8, 8))
    e.Conv2dMaxPool(tx, tw0, p0, (1, 1), bias=tb0, act="leaky", alpha=0.1)
    e.Conv2dMaxPool(p0, tw1, p1, (1, 1), bias=tb1, act="rectify")
    e.Conv2d(p1, tw2, y2, (1, 1), bias=tb2)
    assert e.conv2d_path(p0, tw1, (1, 1)) == _lib.CONV_TC_WINDOW and e.conv2d_path(p1, tw2, (1, 1)) == _lib.CONV_TC_TMA
    # chained: no NCHW tensor between the links; the second link also keeps an NCHW copy, to be compared
    s0 = (e.empty((B, 16, 16, 32)), e.empty((B, 16, 16, 32)))
    s1 = (e.empty((B, 8, 8, 64)), e.empty((B, 8, 8, 64)))
    q1, z2 = e.empty((B, 64, 8, 8)), e.empty((B, 40, 8, 8))
    e.Conv2dChain(tx, tw0, None, (B, 3, 32, 32), (1, 1), bias=tb0, act="leaky", alpha=0.1, pool2=True, y_split=s0)
    e.Conv2dChain(None, tw1, q1, (B, 32, 16, 16), (1, 1), bias=tb1, act="rectify", pool2=True, x_split=s0, y_split=s1)
    e.Conv2dChain(None, tw2, z2, (B, 64, 8, 8), (1, 1), bias=tb2, x_split=s1)
    assert_bits_equal(q1.numpy(), p1.numpy())
    assert_bits_equal(z2.numpy(), y2.numpy())
    # the split form itself: head + tail reproduce the NCHW tensor to 2^-21, head is its TF32 rounding
    nhwc = np.transpose(p1.numpy(), (0, 2, 3, 1))
    hi, lo = s1[0].numpy(), s1[1].numpy()
    assert np.all((hi.view(np.uint32) & 0x1FFF) == 0)
    assert np.abs((hi.astype(np.float64) + lo) - nhwc).max() <= 2.0 ** -21 * max(1.0, float(np.abs(nhwc).max()))


def test_conv2d_chain_fallbacks(fresh):
    from gorgonia_b200 import B200Error, _lib
    e = fresh
    # a link whose kernel reads NCHW (8 channels: gather path) still delivers the split form, by a rewrite pass
    B = 12
    x = util.uniform(108, (B, 8, 24, 24)) - np.float32(0.5)
    w = util.normal(109, (32, 8, 3, 3), scale=0.2)
    w2 = util.normal(110, (16, 32, 3, 3), scale=0.1)
    tx, tw, tw2 = e.tensor(x), e.tensor(w), e.tensor(w2)
    assert e.conv2d_path(tx, tw, (1, 1)) == _lib.CONV_TC_GATHER
    p = e.empty((B, 32, 12, 12))
    e.Conv2dMaxPool(tx, tw, p, (1, 1), act="rectify")
    ref = e.empty((B, 16, 12, 12))
    e.Conv2d(p, tw2, ref, (1, 1))
    sp = (e.empty((B, 12, 12, 32)), e.empty((B, 12, 12, 32)))
    got = e.empty((B, 16, 12, 12))
    e.Conv2dChain(tx, tw, None, (B, 8, 24, 24), (1, 1), act="rectify", pool2=True, y_split=sp)
    e.Conv2dChain(None, tw2, got, (B, 32, 12, 12), (1, 1), x_split=sp)
    assert_bits_equal(got.numpy(), ref.numpy())
    # without the NCHW input such a link cannot run
    with pytest.raises(B200Error) as ei:
        e.Conv2dChain(None, tw, p, (B, 8, 24, 24), (1, 1), x_split=sp)
    assert ei.value.code == _lib.ERR_UNSUPPORTED


def test_conv2d_matches_reference_pipeline(fresh):
    # Conv2d as gorgonia spells it (nn.go:264-298): Im2Col -> MatMul(transB) -> Transpose(0,3,1,2)
    e = fresh
    B, Cc, H, W, K = 2, 3, 9, 8, 5
    x, w = util.uniform(1, (B, Cc, H, W)), util.normal(2, (K, Cc, 3, 3))
    tx, tw = e.tensor(x), e.tensor(w)
    col = e.empty((B, H, W, Cc * 9))
    e.Im2Col(tx, col, (3, 3), (1, 1))
    assert_bits_equal(col.numpy(), oracle.im2col(x, 3, 3, (1, 1)))
    prod = e.empty((B * H * W, K))
    e.MatMul(col.reshape(B * H * W, Cc * 9), tw.reshape(K, Cc * 9), prod, transB=True)
    out = e.empty((B, K, H, W))
    e.Transpose(prod.reshape(B, H, W, K), out, (0, 3, 1, 2))
    fused = e.empty((B, K, H, W))
    e.Conv2d(tx, tw, fused, (1, 1))
    assert_gemm_close(out.numpy(), oracle.conv2d(x, w, (1, 1)), 1e-5)
    assert_gemm_close(fused.numpy(), out.numpy(), 1e-5)


def test_im2col_variants(fresh):
    e = fresh
    for (B, Cc, H, W, kh, kw, pad, stride, dil) in [(2, 3, 7, 6, 3, 3, (1, 1), (1, 1), (1, 1)),
                                                    (1, 2, 9, 9, 2, 4, (0, 2), (2, 1), (1, 1)),
                                                    (2, 1, 10, 10, 3, 3, (2, 2), (1, 1), (2, 2))]:
        x = util.normal(3, (B, Cc, H, W))
        want = oracle.im2col(x, kh, kw, pad, stride, dil)
        col = e.empty(want.shape)
        e.Im2Col(e.tensor(x), col, (kh, kw), pad, stride, dil)
        assert_bits_equal(col.numpy(), want)


POOL_CASES = [
    ((2, 3, 28, 28), (2, 2), (0, 0), (2, 2)),
    ((2, 3, 7, 7), (2, 2), (0, 0), (2, 2)),            # 7 -> 3: the last row and column are dropped
    ((1, 2, 13, 13), (2, 2), (1, 0, 1, 0), (1, 1)),    # tiny-YOLO's last pool: explicit padding, 13 -> 13
    ((1, 1, 4, 4), (2, 2), (0, 0), (1, 1)),
    ((2, 2, 9, 11), (3, 2), (1, 1), (2, 3)),
    ((1, 1, 5, 5), (3, 3), (0, 1, 1, 0), (2, 2)),
]


@pytest.mark.parametrize("shape,kernel,pad,stride", POOL_CASES)
def test_maxpool(fresh, shape, kernel, pad, stride):
    e = fresh
    x = util.normal(5, shape)
    x[0, 0, 0, :2] = 3.0                    # a tie inside the first window
    want, wmask = oracle.maxpool2d(x, kernel, pad, stride)
    y, mask = e.empty(want.shape), e.empty(want.shape, np.int64)
    e.MaxPool2D(e.tensor(x), y, kernel, pad, stride, mask=mask)
    assert_bits_equal(y.numpy(), want)
    assert np.array_equal(mask.numpy(), wmask)


def test_maxpool_all_nan_window(fresh):
    e = fresh
    x = np.full((1, 1, 2, 2), np.nan, np.float32)
    y = e.empty((1, 1, 1, 1))
    e.MaxPool2D(e.tensor(x), y, (2, 2), (0, 0), (2, 2))
    assert y.numpy().item() == -np.finfo(np.float32).max      # op_nn.go:862,890: nothing beats -MaxFloat32


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.int64])
@pytest.mark.parametrize("shape,perm", [((3, 5), (1, 0)), ((2, 3, 4), (2, 0, 1)), ((4, 6, 5, 7), (0, 3, 1, 2)),
                                        ((4, 6, 5, 7), (0, 2, 3, 1)), ((2, 3, 4, 5), (3, 2, 1, 0)),
                                        ((100, 257), (1, 0)), ((1, 7, 1, 9), (3, 2, 1, 0)), ((6,), (0,)),
                                        ((3, 4, 5), (0, 1, 2))])
def test_transpose(fresh, shape, perm, dt):
    e = fresh
    x = (util.normal(6, shape, np.float64) * 100).astype(dt)
    want = oracle.transpose(x, perm)
    y = e.empty(want.shape, dt)
    e.Transpose(e.tensor(x), y, perm)
    assert np.array_equal(y.numpy(), want)
    assert np.array_equal(want, np.transpose(x, perm))


def test_by_indices(fresh):
    from gorgonia_b200 import B200Error
    e = fresh
    for shape in [(10, 4), (33, 7), (5, 3, 2), (100,)]:
        x = util.normal(7, shape)
        idx = util.rng(8).integers(0, shape[0], size=17).astype(np.int64)
        y = e.empty((17,) + shape[1:])
        e.ByIndices(e.tensor(x), e.tensor(idx), y)
        assert_bits_equal(y.numpy(), oracle.gather_rows(x, idx))
    with pytest.raises(B200Error):
        e.ByIndices(e.tensor(x), e.tensor(np.array([0, 100], np.int64)), e.empty((2,)))


@pytest.mark.parametrize("case", [((3, 40, 13, 13), (2, 2), (1, 0, 1, 0), (1, 1)),     # tiny-YOLO's stride-1 pool
                                  ((2, 64, 52, 52), (2, 2), (0, 0), (2, 2)),
                                  ((2, 33, 9, 11), (3, 3), (1, 1), (2, 2))])            # ragged channel / position tiles
def test_maxpool_split_form(fresh, case):
    # the pool that feeds a convolution chain writes NCHW (optional) and the NHWC TF32 head/tail pair
    e = fresh
    shape, kernel, pad, stride = case
    x = util.normal(130, shape)
    want, _ = oracle.maxpool2d(x, kernel, pad, stride)
    B, Cc, Ho, Wo = want.shape
    y, hi, lo = e.empty(want.shape), e.empty((B, Ho, Wo, Cc)), e.empty((B, Ho, Wo, Cc))
    e.MaxPool2DSplit(e.tensor(x), y, (hi, lo), kernel, pad, stride)
    assert_bits_equal(y.numpy(), want)
    nhwc = np.transpose(want, (0, 2, 3, 1))
    h, l = hi.numpy(), lo.numpy()
    assert np.all((h.view(np.uint32) & 0x1FFF) == 0) and np.all((l.view(np.uint32) & 0x1FFF) == 0)
    assert np.abs((h.astype(np.float64) + l) - nhwc).max() <= 2.0 ** -21 * float(np.abs(nhwc).max())
    # without the NCHW copy
    hi2, lo2 = e.empty((B, Ho, Wo, Cc)), e.empty((B, Ho, Wo, Cc))
    e.MaxPool2DSplit(e.tensor(x), None, (hi2, lo2), kernel, pad, stride)
    assert_bits_equal(hi2.numpy(), h)
    assert_bits_equal(lo2.numpy(), l)

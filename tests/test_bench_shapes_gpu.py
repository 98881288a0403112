"""Parity at the shapes bench.py times (GPU tests).

The small-shape tests elsewhere in this folder pick narrow tiles and give every persistent CTA at
most one tile. The shapes here select the kernel instantiations the benchmark runs (128- and
256-column tiles, all 512 columns of tensor memory), make every CTA walk several tiles and several
raster groups, and run the graphs at their benchmark batch sizes. Where the oracle would need
minutes for the whole result, it computes a sample that touches every tile (one row and one column
per 128-wide tile) and a whole-result property closes the gap:

  - matrix products: (A.B).v == A.(B.v) for a random sign vector v, evaluated in double on the host,
    which no skipped, repeated or misplaced tile survives;
  - graphs: the batch is a small set of distinct images repeated, and every repetition is held to
    the oracle's result for its original (a launch that shares tiles' k ranges between CTAs sums
    different tiles in different groupings, so repetitions agree within the tolerance, not bit for
    bit).

Tolerances as everywhere: 1e-5 * max(|r|, rms(r)) for float32 products, 1e-2 on that scale for
bfloat16 operands, bit-exact for Outer."""
import numpy as np
import pytest

from gorgonia_b200 import tapes
from gorgonia_b200.engine import from_bf16, to_bf16
from oracle import graphs, oracle
from tests import util
from tests.util import assert_bits_equal, assert_gemm_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def big():
    """An engine with a 20 GiB arena: the benchmark shapes do not fit the session engine's 4 GiB."""
    from gorgonia_b200 import Engine
    e = Engine(device=0, arena_bytes=20 << 30)
    yield e
    e.Close()


@pytest.fixture()
def roomy(big):
    big.ResetAllocator()
    yield big
    big.Signal()
    big.ResetAllocator()


def _sampled_product_check(got, a, b, rel, tile=128):
    """got = a @ b on the device. One row and one column per tile against the oracle, then the
    probe-vector identity over the whole result."""
    M, N = got.shape
    g = util.rng(991)
    rows = np.array([min(M - 1, t * tile + int(g.integers(tile))) for t in range((M + tile - 1) // tile)])
    cols = np.array([min(N - 1, t * tile + int(g.integers(tile))) for t in range((N + tile - 1) // tile)])
    want_rows = oracle.gemm(np.ascontiguousarray(a[rows]), b)
    want_cols = oracle.gemm(a, np.ascontiguousarray(b[:, cols]))
    rms = float(np.sqrt(np.mean(want_rows.astype(np.float64) ** 2)))
    for gs, ws in ((got[rows], want_rows), (got[:, cols], want_cols)):
        err = np.abs(gs.astype(np.float64) - ws)
        lim = rel * np.maximum(np.abs(ws.astype(np.float64)), rms)
        assert (err <= lim).all(), f"sampled product off by {float((err / lim).max()):.3g} x tolerance"
    v = g.integers(0, 2, N).astype(np.float64) * 2 - 1
    lhs = got.astype(np.float64) @ v
    rhs = a.astype(np.float64) @ (b.astype(np.float64) @ v)
    # every element within rel * rms moves a row sum by at most rel * rms * N; a lost 128-wide tile
    # moves it by about rms * sqrt(128)
    assert np.abs(lhs - rhs).max() <= rel * rms * N, "probe-vector identity violated: a tile is wrong"


@pytest.mark.parametrize("shape", [(2304, 2304, 512), (4096, 4096, 4096), (8192, 8192, 8192)])
def test_matmul_f32_wide_tiles_many_per_cta(roomy, shape):
    # 128-column tiles (the instantiation that owns all 512 tensor-memory columns): 324 / 1024 / 4096
    # tiles over 148 persistent CTAs, 3 / 4 / 8 raster groups with 18 / 32 / 64 column tiles each
    e = roomy
    M, N, K = shape
    a = util.normal(300 + M, (M, K), scale=0.02)
    b = util.normal(301 + M, (K, N), scale=0.02)
    ta, tb, tc = e.tensor(a), e.tensor(b), e.empty((M, N))
    assert e.gemm_path(ta, tb, tc) == 1
    e.MatMul(ta, tb, tc)
    got = tc.numpy()
    if M <= 2304:
        assert_gemm_close(got, oracle.gemm(a, b), 1e-5)
    _sampled_product_check(got, a, b, 1e-5)


def test_matmul_f32_ragged_last_wave(roomy):
    # 85 x 8 = 680 tiles on 148 SMs: four full waves of whole tiles, then 88 tiles whose k range is shared out
    # over all CTAs (the launch shape of tiny-YOLO's late layers at the benchmark batch)
    e = roomy
    M, N, K = 10880, 1024, 1024
    a = util.normal(305, (M, K), scale=0.02)
    b = util.normal(306, (K, N), scale=0.02)
    ta, tb, tc = e.tensor(a), e.tensor(b), e.empty((M, N))
    e.MatMul(ta, tb, tc)
    got = tc.numpy()
    _sampled_product_check(got, a, b, 1e-5)
    # an engine that never shares k ranges agrees within the tolerance (not bit for bit: the shared tiles
    # are summed in other groupings)
    from gorgonia_b200 import Engine
    e2 = Engine(device=0, arena_bytes=1 << 30, streamk=False)
    ua, ub, uc = e2.tensor(a), e2.tensor(b), e2.empty((M, N))
    e2.MatMul(ua, ub, uc)
    assert_gemm_close(got, uc.numpy(), 1e-5)
    e2.Close()


def test_matmul_f32_incr_4096(roomy):
    # the Incr-mode benchmark shape: C += A.B equals MatMul followed by Add, bit for bit
    e = roomy
    n = 4096
    a, b = util.normal(310, (n, n), scale=0.02), util.normal(311, (n, n), scale=0.02)
    c0 = util.normal(312, (n, n), scale=0.1)
    ta, tb, tc, tp = e.tensor(a), e.tensor(b), e.tensor(c0), e.empty((n, n))
    e.MatMul(ta, tb, tc, incr=True)
    e.MatMul(ta, tb, tp)
    e.Add(tp, e.tensor(c0), unsafe=True)
    assert_bits_equal(tc.numpy(), tp.numpy())


@pytest.mark.parametrize("shape,tile", [((1536, 1792, 512), 128), ((2048, 2560, 512), 256), ((4096, 4096, 4096), 256),
                                        ((8192, 8192, 8192), 256)])
def test_matmul_bf16_wide_tiles(roomy, shape, tile):
    # 128-column tiles: 12 x 14 = 168 tiles; 256-column tiles: 16 x 10 = 160, 32 x 16 = 512, 64 x 32 = 2048
    e = roomy
    M, N, K = shape
    a = from_bf16(to_bf16(util.normal(320 + M, (M, K), scale=0.02)))
    b = from_bf16(to_bf16(util.normal(321 + M, (K, N), scale=0.02)))
    ta, tb, tc = e.tensor_bf16(a), e.tensor_bf16(b), e.empty((M, N))
    e.MatMul(ta, tb, tc)
    got = tc.numpy()
    if M <= 2048:
        assert_gemm_close(got, oracle.gemm(a, b), 1e-4)
    _sampled_product_check(got, a, b, 1e-4, tile=128)


@pytest.mark.parametrize("transA,transB", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(4096, 4864, 256), (3992, 4872, 192)])
def test_matmul_bf16_cta_pairs(shape, transA, transB):
    # 16 x 19 tiles of 256 x 256 (the second shape ragged in rows and columns) are enough for the launch
    # to run as pairs of CTAs on 256-row tiles (cluster of two, tcgen05 cta_group::2): against the oracle,
    # and bit for bit against an engine that never pairs CTAs up, in all four operand layouts
    from gorgonia_b200 import Engine
    M, N, K = shape
    a = from_bf16(to_bf16(util.normal(325, (K, M) if transA else (M, K), scale=0.02)))
    b = from_bf16(to_bf16(util.normal(326, (N, K) if transB else (K, N), scale=0.02)))
    got = {}
    for pairs in (True, False):
        e = Engine(device=0, arena_bytes=1 << 30, pairs=pairs)
        ta, tb, tc = e.tensor_bf16(a), e.tensor_bf16(b), e.empty((M, N))
        e.MatMul(ta, tb, tc, transA, transB)
        got[pairs] = tc.numpy()
        e.Close()
    assert_bits_equal(got[True], got[False])
    assert_gemm_close(got[True], oracle.gemm(a, b, transA, transB), 1e-4)


@pytest.mark.parametrize("bf16", [False, True])
def test_batch_of_64_products_512(roomy, bf16):
    e = roomy
    A = util.normal(330, (64, 512, 512), scale=0.02)
    B = util.normal(331, (64, 512, 512), scale=0.02)
    if bf16:
        A, B = from_bf16(to_bf16(A)), from_bf16(to_bf16(B))
        ta, tb = e.tensor_bf16(A), e.tensor_bf16(B)
    else:
        ta, tb = e.tensor(A), e.tensor(B)
    out = e.empty((64, 512, 512))
    e.MatMul(ta, tb, out)
    assert_gemm_close(out.numpy(), oracle.batched_matmul(A, B), 1e-4 if bf16 else 1e-5)


def test_matvecmul_16384(roomy):
    e = roomy
    n = 16384
    a = util.normal(340, (n, n), scale=0.02)
    x = util.normal(341, n)
    ta, y = e.tensor(a), e.empty(n)
    e.MatVecMul(ta, e.tensor(x), y)
    assert_gemm_close(y.numpy(), oracle.gemv(a, x), 1e-5)
    e.MatVecMul(ta, e.tensor(x), y, transA=True)
    assert_gemm_close(y.numpy(), oracle.gemv(a, x, transA=True), 1e-5)


def test_outer_8192(roomy):
    e = roomy
    x, y = util.normal(350, 8192), util.normal(351, 8192)
    out = e.empty((8192, 8192))
    e.Outer(e.tensor(x), e.tensor(y), out)
    assert_bits_equal(out.numpy(), oracle.outer(x, y))


@pytest.mark.parametrize("case", [
    # (input shape, output channels, expected kernel): more tiles than the GPU has SMs
    ((8, 64, 52, 52), 128, "tma"),      # 169 tiles of 128 positions
    ((3, 256, 26, 26), 512, "tma"),     # 16 position tiles x 4 channel tiles, ragged last position tile
    ((16, 32, 64, 64), 64, "window"),   # 256 window tiles
    ((40, 32, 14, 14), 64, "window"),   # LeNet conv1's plane: 16 x 16 tiles hang over a 14 x 14 image
])
def test_convolution_many_tiles_per_cta(roomy, case):
    from gorgonia_b200 import _lib
    e = roomy
    shape, K, kind = case
    x = util.uniform(360 + shape[1], shape) - np.float32(0.5)
    w = util.normal(361, (K, shape[1], 3, 3), scale=0.1)
    bias = util.normal(362, K, scale=0.1)
    tx, tw, tb = e.tensor(x), e.tensor(w), e.tensor(bias)
    assert e.conv2d_path(tx, tw, (1, 1)) == {"tma": _lib.CONV_TC_TMA, "window": _lib.CONV_TC_WINDOW}[kind]
    y = e.empty((shape[0], K, shape[2], shape[3]))
    e.Conv2d(tx, tw, y, pad=(1, 1), bias=tb, act="leaky", alpha=0.1)
    want = oracle.leaky_relu((oracle.conv2d(x, w, (1, 1)) + bias[None, :, None, None]).astype(np.float32), 0.1)
    assert_gemm_close(y.numpy(), want, 1e-5)


def test_lenet_at_benchmark_batch(roomy):
    # 64 distinct images repeated 128 times: the oracle checks the 64, every repetition must match
    e = roomy
    B = 8192
    x64 = util.uniform(370, (64, 1, 28, 28))
    m = tapes.LeNet(e, B)
    m.x.set(np.tile(x64, (B // 64, 1, 1, 1)))
    got = m.forward().numpy()
    want = graphs.lenet(m, x64)
    assert_gemm_close(got.reshape(B // 64, 64, 10), np.broadcast_to(want, (B // 64, 64, 10)), 1e-5)
    assert np.array_equal(got.reshape(B // 64, 64, 10).argmax(2), np.broadcast_to(want.argmax(1), (B // 64, 64)))
    # and 64 images spread over the batch with nothing repeated
    xr = util.uniform(371, (B, 1, 28, 28))
    m.x.set(xr)
    got = m.forward().numpy()
    idx = np.arange(64) * 128 + util.rng(372).integers(0, 128, 64)
    assert_gemm_close(got[idx], graphs.lenet(m, xr[idx]), 1e-5)
    # the recorded tape gives the same bits at this size
    m.record()
    m.replay()
    assert_bits_equal(m.out.numpy(), got)
    m.close()


def test_tiny_yolo_at_benchmark_batch(roomy):
    # two distinct 416 x 416 images repeated 32 times
    e = roomy
    B = 64
    x2 = util.uniform(380, (2, 3, 416, 416))
    m = tapes.TinyYolo(e, B)
    m.x.set(np.tile(x2, (B // 2, 1, 1, 1)))
    got = m.forward().numpy()
    assert got.shape == (B, 125, 13, 13)
    want = graphs.tiny_yolo(m, x2)
    assert_gemm_close(got.reshape(B // 2, 2, 125, 13, 13), np.broadcast_to(want, (B // 2, 2, 125, 13, 13)), 1e-5)
    m.record()
    m.replay()
    assert_bits_equal(m.out.numpy(), got)
    m.close()


def test_tiny_yolo_small_shards(roomy):
    # the per-GPU batches of the 8- and 4-GPU runs: the late layers have fewer tiles than SMs there
    e = roomy
    x2 = util.uniform(381, (2, 3, 416, 416))
    ref = None
    for B in (8, 16):
        m = tapes.TinyYolo(e, B)
        m.x.set(np.tile(x2, (B // 2, 1, 1, 1)))
        got = m.forward().numpy()
        if ref is None:
            ref = graphs.tiny_yolo(m, x2)
        assert_gemm_close(got.reshape(B // 2, 2, 125, 13, 13), np.broadcast_to(ref, (B // 2, 2, 125, 13, 13)), 1e-5)
        e.Signal()
        e.ResetAllocator()

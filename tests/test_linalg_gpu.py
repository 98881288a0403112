"""Parity of MatMul / MatVecMul / Outer / batched MatMul against the CPU oracle (GPU tests).

Tolerance: |g - r| <= 1e-5 * max(|r|, rms(r)) for float32 (the oracle accumulates in double),
1e-2 on the same scale for bfloat16 operands (whose oracle is fed the bf16-rounded inputs, so
the tolerance covers accumulation only), 1e-12 for float64."""
import numpy as np
import pytest

from gorgonia_b200.engine import from_bf16, to_bf16
from oracle import oracle
from tests import util
from tests.util import assert_bits_equal, assert_gemm_close

pytestmark = pytest.mark.gpu


def _mats(seed, M, N, K, transA, transB, dt=np.float32, scale=0.02):
    a = util.normal(seed, (K, M) if transA else (M, K), dt, scale)
    b = util.normal(seed + 1, (N, K) if transB else (K, N), dt, scale)
    return a, b


TC_SHAPES = [(128, 128, 64), (256, 256, 256), (1024, 1024, 1024), (200, 328, 136), (130, 70, 40), (64, 1000, 512),
             (1, 512, 512), (777, 33, 1001), (256, 300, 784), (4096, 64, 27),
             (512, 10, 625), (300, 3, 512)]


@pytest.mark.parametrize("transA,transB", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", TC_SHAPES)
def test_matmul_f32_tensor_core_path(fresh, shape, transA, transB):
    e = fresh
    M, N, K = shape
    a, b = _mats(100 + M + N, M, N, K, transA, transB)
    ta, tb, tc = e.tensor(a), e.tensor(b), e.empty((M, N))
    assert e.gemm_path(ta, tb, tc, transA, transB) == 1      # tcgen05 kernel, not the CUDA-core one
    e.MatMul(ta, tb, tc, transA, transB)
    e.Signal()
    assert_gemm_close(tc.numpy(), oracle.gemm(a, b, transA, transB), 1e-5)


@pytest.mark.parametrize("transA,transB", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (512, 512, 512), (304, 264, 200), (1024, 2048, 768)])
def test_matmul_bf16(fresh, shape, transA, transB):
    e = fresh
    M, N, K = shape
    a, b = _mats(7 + M, M, N, K, transA, transB)
    ta, tb, tc = e.tensor_bf16(a), e.tensor_bf16(b), e.empty((M, N))
    assert e.gemm_path(ta, tb, tc, transA, transB) == 1
    e.MatMul(ta, tb, tc, transA, transB)
    e.Signal()
    want = oracle.gemm(from_bf16(to_bf16(a)), from_bf16(to_bf16(b)), transA, transB)
    assert_gemm_close(tc.numpy(), want, 1e-2)
    # bf16 products are exact in fp32 and the accumulator is fp32: far inside the bf16 budget
    assert_gemm_close(tc.numpy(), want, 1e-4)


def test_matmul_bf16_unaligned_pitch_is_refused(fresh):
    # TMA reads bf16 operands in place: a row pitch that is not a multiple of 16 bytes is an error,
    # not a silent detour through another kernel
    from gorgonia_b200 import B200Error
    e = fresh
    a, b = _mats(1, 128, 128, 100, False, False)       # pitch of A = 100 * 2 bytes
    with pytest.raises(B200Error) as ei:
        e.MatMul(e.tensor_bf16(a), e.tensor_bf16(b), e.empty((128, 128)))
    assert ei.value.code == 4


def test_matmul_large_k_accuracy(fresh):
    # K = 8192 sums: the 3xTF32 split has to hold 1e-5 where plain TF32 (~1e-3) cannot
    e = fresh
    M, N, K = 256, 256, 8192
    a, b = _mats(5, M, N, K, False, False)
    ta, tb, tc = e.tensor(a), e.tensor(b), e.empty((M, N))
    e.MatMul(ta, tb, tc)
    want = oracle.gemm(a, b)
    assert_gemm_close(tc.numpy(), want, 1e-5)
    # for scale: a float32 BLAS that sums in k order differs from the double oracle by this much
    naive = oracle.gemm_f32_naive(a, b)
    rms = np.sqrt(np.mean(want.astype(np.float64) ** 2))
    print("3xTF32 max err/rms", np.abs(tc.numpy() - want).max() / rms, "fp32 k-order err/rms",
          np.abs(naive - want).max() / rms)


@pytest.mark.parametrize("shape", [(5, 7, 3), (2, 2, 2), (63, 10, 100), (256, 10, 100), (31, 15, 1)])
@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_matmul_cuda_core_path(fresh, shape, dt):
    e = fresh
    M, N, K = shape
    for transA, transB in [(False, False), (True, False), (False, True), (True, True)]:
        a, b = _mats(3 + M, M, N, K, transA, transB, dt, 1.0)
        ta, tb, tc = e.tensor(a), e.tensor(b), e.empty((M, N), dt)
        e.MatMul(ta, tb, tc, transA, transB)
        assert_gemm_close(tc.numpy(), oracle.gemm(a, b, transA, transB), 1e-5 if dt == np.float32 else 1e-12)


def test_matmul_f64_large(fresh):
    e = fresh
    a, b = _mats(9, 300, 200, 150, False, False, np.float64, 1.0)
    tc = e.empty((300, 200), np.float64)
    e.MatMul(e.tensor(a), e.tensor(b), tc)
    assert_gemm_close(tc.numpy(), oracle.gemm(a, b), 1e-12)


def test_matmul_fused_epilogue(fresh):
    e = fresh
    M, N, K = 256, 300, 784
    a, b = _mats(11, M, N, K, False, False, scale=0.05)
    bias = util.normal(12, N, scale=0.05)
    ta, tb, tbias, tc = e.tensor(a), e.tensor(b), e.tensor(bias), e.empty((M, N))
    e.MatMul(ta, tb, tc, bias=tbias, bias_kind="col", act="rectify")
    plain = e.empty((M, N))
    e.MatMul(ta, tb, plain)
    # the fused store equals the unfused engine sequence bit for bit
    e.BroadcastBinary("add", plain, tbias, 1, N, unsafe=True)
    mask = e.empty((M, N))
    e.GteScalar(plain, 0.0, reuse=mask)
    e.Mul(plain, mask, unsafe=True)
    assert_bits_equal(tc.numpy(), plain.numpy())
    want = oracle.rectify((oracle.gemm(a, b) + bias[None, :]).astype(np.float32))
    assert_gemm_close(tc.numpy(), want, 1e-5)
    # leaky, per-row bias, CUDA-core path
    M2, N2, K2 = 20, 12, 9
    a2, b2 = _mats(13, M2, N2, K2, False, False, scale=1.0)
    rb = util.normal(14, M2)
    t2 = e.empty((M2, N2))
    e.MatMul(e.tensor(a2), e.tensor(b2), t2, bias=e.tensor(rb), bias_kind="row", act="leaky", alpha=0.1)
    want2 = oracle.leaky_relu((oracle.gemm(a2, b2) + rb[:, None]).astype(np.float32), 0.1)
    assert_gemm_close(t2.numpy(), want2, 1e-5)


def test_batched_matmul(fresh):
    # golden of gorgonia's binOpTests (op_math_test.go:347-358) plus random batches
    e = fresh
    a = np.tile(np.arange(1, 13, dtype=np.float64), 2).reshape(2, 3, 4)
    b = np.tile(np.arange(1, 5, dtype=np.float64), 2).reshape(2, 4, 1)
    tc = e.empty((2, 3, 1), np.float64)
    e.MatMul(e.tensor(a), e.tensor(b), tc)
    assert tc.numpy().reshape(-1).tolist() == [30, 70, 110, 30, 70, 110]
    for transA, transB in [(False, False), (False, True), (True, False)]:
        A = util.normal(21, (4, 3, 192, 136) if transA else (4, 3, 136, 192), scale=0.1)
        Bm = util.normal(22, (4, 3, 96, 192) if transB else (4, 3, 192, 96), scale=0.1)
        out = e.empty((4, 3, 136, 96))
        e.MatMul(e.tensor(A), e.tensor(Bm), out, transA, transB)
        assert_gemm_close(out.numpy(), oracle.batched_matmul(A, Bm, transA, transB), 1e-5)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("shape", [(1, 1), (3, 5), (128, 128), (1000, 257), (513, 4096), (4100, 31),
                                   (300, 4100), (9, 8196), (21, 20484)])   # long rows: x shared through shared memory
def test_matvecmul(fresh, shape, dt):
    e = fresh
    M, N = shape
    a = util.normal(31, (M, N), dt)
    tol = 1e-5 if dt == np.float32 else 1e-12
    x = util.normal(32, N, dt)
    y = e.empty(M, dt)
    e.MatVecMul(e.tensor(a), e.tensor(x), y)
    assert_gemm_close(y.numpy(), oracle.gemv(a, x), tol)
    xt = util.normal(33, M, dt)
    yt = e.empty(N, dt)
    e.MatVecMul(e.tensor(a), e.tensor(xt), yt, transA=True)
    assert_gemm_close(yt.numpy(), oracle.gemv(a, xt, transA=True), tol)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_outer(fresh, dt):
    e = fresh
    for M, N in [(1, 1), (3, 5), (64, 64), (1000, 1031), (257, 4096)]:
        x, y = util.normal(41, M, dt), util.normal(42, N, dt)
        out = e.tensor(np.full((M, N), 7.0, dt))           # overwritten, not accumulated into
        e.Outer(e.tensor(x), e.tensor(y), out)
        assert_bits_equal(out.numpy(), oracle.outer(x, y))
        out.free()


def test_gemm_argument_errors(fresh):
    from gorgonia_b200 import B200Error
    e = fresh
    a, b = e.tensor(np.ones((4, 5), np.float32)), e.tensor(np.ones((6, 7), np.float32))
    with pytest.raises(B200Error):
        e.MatMul(a, b, e.empty((4, 7)))


def test_constant_operand_split_is_kept_until_undeclared(fresh):
    # weights declared constant are split once; the engine must not notice a change of their
    # contents until the declaration is withdrawn (that is the documented contract)
    e = fresh
    M, N, K = 256, 128, 192
    a, b = _mats(71, M, N, K, False, False, scale=0.1)
    ta, tb, tc = e.tensor(a), e.tensor(b), e.empty((M, N))
    e.Signal()
    e.constant(tb)
    l0 = e.launches
    e.MatMul(ta, tb, tc)
    first = e.launches - l0
    want = oracle.gemm(a, b)
    assert_gemm_close(tc.numpy(), want, 1e-5)
    l0 = e.launches
    e.MatMul(ta, tb, tc)
    assert e.launches - l0 == first - 1            # the split of B was not repeated
    assert_gemm_close(tc.numpy(), want, 1e-5)
    b2 = (b * np.float32(2.0)).astype(np.float32)
    tb.set(b2)
    e.constant(tb, False)                          # withdrawn: the next product sees the new values
    e.MatMul(ta, tb, tc)
    assert_gemm_close(tc.numpy(), oracle.gemm(a, b2), 1e-5)
    used = e.arena_stats()["used"]
    e.constant(tb)
    e.MatMul(ta, tb, tc)
    assert e.arena_stats()["used"] > used          # the kept split lives in the arena ...
    tb.free()
    assert e.arena_stats()["used"] < used          # ... and goes with the buffer it was derived from


def test_matmul_chain_equals_the_unchained_calls(fresh):
    # three dense layers; the activations between them exist only as TF32 head/tail pairs written by
    # the producing link's epilogue. Bit-equal to MatMul with the same fused bias / activation.
    e = fresh
    M, dims = 512, (784, 300, 100, 64)
    x = util.normal(201, (M, dims[0]))
    ws = [util.normal(202 + i, (dims[i], dims[i + 1]), scale=0.05) for i in range(3)]
    bs = [util.normal(210 + i, dims[i + 1], scale=0.1) for i in range(3)]
    tx, tw, tb = e.tensor(x), [e.tensor(w) for w in ws], [e.tensor(b) for b in bs]
    h = [e.empty((M, d)) for d in dims[1:]]
    a = tx
    for i in range(3):
        e.MatMul(a, tw[i], h[i], bias=tb[i], bias_kind="col", act="rectify" if i < 2 else None)
        a = h[i]
    s0 = (e.empty((M, 300)), e.empty((M, 300)))
    s1 = (e.empty((M, 100)), e.empty((M, 100)))
    keep1, out = e.empty((M, 100)), e.empty((M, 64))
    e.MatMulChain(tx, tw[0], None, M, 300, 784, bias=tb[0], act="rectify", c_split=s0, ld_split=300)
    e.MatMulChain(None, tw[1], keep1, M, 100, 300, bias=tb[1], act="rectify", a_split=s0, c_split=s1, ld_split=100)
    e.MatMulChain(None, tw[2], out, M, 64, 100, bias=tb[2], a_split=s1)
    assert_bits_equal(keep1.numpy(), h[1].numpy())
    assert_bits_equal(out.numpy(), h[2].numpy())
    hi, lo = s1[0].numpy(), s1[1].numpy()
    assert np.all((hi.view(np.uint32) & 0x1FFF) == 0)
    assert np.abs((hi.astype(np.float64) + lo) - h[1].numpy()).max() <= 2.0 ** -21 * max(1.0, float(np.abs(h[1].numpy()).max()))


def test_matmul_chain_ragged_pitch_and_fallback(fresh):
    from gorgonia_b200 import B200Error, _lib
    e = fresh
    M, K, N = 300, 200, 625                      # N not a multiple of 4: pitch 628, zero-filled tail columns
    a, b = util.normal(220, (M, K), scale=0.1), util.normal(221, (K, N), scale=0.1)
    b2 = util.normal(222, (N, 40), scale=0.1)
    ta, tb, tb2 = e.tensor(a), e.tensor(b), e.tensor(b2)
    c, ref = e.empty((M, N)), e.empty((M, 40))
    e.MatMul(ta, tb, c, act="rectify")
    e.MatMul(c, tb2, ref)
    sp = (e.tensor(np.full((M, 628), 7.0, np.float32)), e.tensor(np.full((M, 628), 7.0, np.float32)))
    got = e.empty((M, 40))
    e.MatMulChain(ta, tb, None, M, N, K, act="rectify", c_split=sp, ld_split=628)
    e.MatMulChain(None, tb2, got, M, 40, N, a_split=sp)
    assert_bits_equal(got.numpy(), ref.numpy())
    assert np.all(sp[0].numpy()[:, 625:] == 0) and np.all(sp[1].numpy()[:, 625:] == 0)
    # a product too small for the tensor cores needs the unsplit A
    small = e.empty((8, 4))
    with pytest.raises(B200Error) as ei:
        e.MatMulChain(None, e.tensor(util.normal(223, (628, 4))), small, 8, 4, 628, a_split=sp)
    assert ei.value.code == _lib.ERR_UNSUPPORTED

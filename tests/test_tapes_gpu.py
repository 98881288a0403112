"""Whole forward tapes (MLP, LeNet, tiny-YOLOv2) against the CPU oracle running the same graph op by
op, plus the properties the engine promises about them: the fused and the instruction-by-
instruction forms agree bit for bit, and a recorded tape replays to the same bits."""
import numpy as np
import pytest

from gorgonia_b200 import tapes
from oracle import graphs
from tests import util
from tests.util import assert_bits_equal, assert_gemm_close

pytestmark = pytest.mark.gpu


def test_mlp_forward(fresh):
    e = fresh
    x = util.uniform(1, (256, 784))
    m = tapes.MLP(e, 256)
    m.b_host = [util.normal(2 + i, b.shape, scale=0.05) for i, b in enumerate(m.b_host)]   # non-trivial biases
    for t, b in zip(m.b, m.b_host):
        t.set(b)
    m.x.set(x)
    got = m.forward().numpy()
    want = graphs.mlp(m, x)
    assert_gemm_close(got, want, 1e-5)
    assert np.array_equal(got.argmax(1), want.argmax(1))
    # instruction-by-instruction form: same bits
    u = tapes.MLP(e, 256, fused=False)
    for t, b in zip(u.b, m.b_host):
        t.set(b)
    u.x.set(x)
    assert_bits_equal(u.forward().numpy(), got)
    # recorded tape: same bits, one host call, and it follows new inputs
    m.record()
    x2 = util.uniform(3, (256, 784))
    m.x.set(x2)
    before = e.launches
    m.replay()
    assert_bits_equal(m.out.numpy(), tapes_forward_fresh(e, m, x2))
    assert e.launches > before
    m.close()


def tapes_forward_fresh(e, m, x):
    m.x.set(x)
    return m.forward().numpy()


def test_lenet_forward(fresh):
    e = fresh
    B = 24
    x = util.uniform(4, (B, 1, 28, 28))
    m = tapes.LeNet(e, B)
    m.x.set(x)
    got = m.forward().numpy()
    want = graphs.lenet(m, x)
    assert_gemm_close(got, want, 1e-5)
    assert np.array_equal(got.argmax(1), want.argmax(1))
    u = tapes.LeNet(e, B, fused=False)
    u.x.set(x)
    assert_bits_equal(u.forward().numpy(), got)
    m.record()
    m.replay()
    assert_bits_equal(m.out.numpy(), got)
    m.close()


def test_tiny_yolo_forward(fresh):
    e = fresh
    x = util.uniform(5, (2, 3, 128, 128))
    m = tapes.TinyYolo(e, 2, size=128)
    m.x.set(x)
    got = m.forward().numpy()
    want = graphs.tiny_yolo(m, x)
    assert got.shape == (2, 125, 4, 4)
    assert_gemm_close(got, want, 1e-5)
    u = tapes.TinyYolo(e, 2, size=128, fused=False)     # one call per convolution and per pool
    u.x.set(x)
    assert_bits_equal(u.forward().numpy(), got)


def test_recording_refuses_calls_that_wait(fresh):
    from gorgonia_b200 import B200Error
    e = fresh
    a = e.tensor(np.ones(8, np.float32))
    e.Signal()
    e.tape_begin()
    try:
        e.AddScalar(a, 1.0, unsafe=True)
        with pytest.raises(B200Error) as ei:
            e.Signal()
        assert ei.value.code == 6
        with pytest.raises(B200Error):
            a.numpy()
    finally:
        t = e.tape_end()
    assert a.numpy()[0] == 1.0          # recorded, not executed
    e.tape_launch(t)
    e.tape_launch(t)
    assert a.numpy()[0] == 3.0
    e.tape_destroy(t)


def test_tape_owns_its_scratch(fresh):
    # While a tape is recorded the library takes arena scratch (TF32 splits of activations, NHWC copies,
    # pool temporaries) and hands it back; the recorded kernels keep those addresses. Nothing that is
    # allocated after the recording may be given those bytes: fill the rest of the arena with known
    # contents, replay, and require both the fillers and the tape's output untouched.
    from gorgonia_b200 import B200Error
    e = fresh
    for make, xshape, seed in ((lambda: tapes.LeNet(e, 24), (24, 1, 28, 28), 6),
                               (lambda: tapes.MLP(e, 256), (256, 784), 7)):
        m = make()
        x = util.uniform(seed, xshape)
        m.x.set(x)
        want = m.forward().numpy()
        before = e.arena_stats()["used"]
        m.record()
        assert e.arena_stats()["used"] > before          # the tape holds what its kernels write
        fillers, size = [], 64 << 20
        while size >= 4096:                              # exhaust the arena, large blocks first
            try:
                t = e.empty(size // 4)
            except B200Error:
                size //= 2
                continue
            fillers.append((t, size))
        assert e.arena_stats()["free"] < 4096 * 64
        for k, (t, sz) in enumerate(fillers):
            check_fill(e, t, float(k + 1))
        m.x.set(util.uniform(seed + 100, xshape))        # different input: the replay must really run
        m.replay()
        m.x.set(x)
        m.replay()
        assert_bits_equal(m.out.numpy(), want)
        for k, (t, sz) in enumerate(fillers):
            probe = t.numpy()
            assert probe[0] == k + 1 and probe[-1] == k + 1 and probe[len(probe) // 2] == k + 1
            assert float(probe.min()) == k + 1 == float(probe.max())
        held = e.arena_stats()["used"]
        m.close()
        assert e.arena_stats()["used"] < held            # destroying the tape gives its blocks back
        for t, _ in fillers:
            t.free()
        e.Signal()
        e.ResetAllocator()


def check_fill(e, t, value):
    t.set(np.full(t.size, value, np.float32))


def test_released_constant_stays_alive_for_its_tape(fresh):
    # what the engine derived from a constant buffer (the TF32 split of a weight matrix) is read by the
    # recorded kernels; withdrawing the declaration afterwards must not free it under the tape
    e = fresh
    a, b = util.normal(60, (256, 192), scale=0.1), util.normal(61, (192, 128), scale=0.1)
    ta, tb, tc = e.tensor(a), e.constant(e.tensor(b)), e.empty((256, 128))
    e.MatMul(ta, tb, tc)
    want = tc.numpy()
    e.tape_begin()
    e.MatMul(ta, tb, tc)
    t = e.tape_end()
    e.constant(tb, False)
    junk = [e.tensor(np.full(192 * 128, 9.0, np.float32)) for _ in range(8)]   # would land on the freed split
    tc.set(np.zeros((256, 128), np.float32))
    e.tape_launch(t)
    assert_bits_equal(tc.numpy(), want)
    e.tape_destroy(t)
    assert len(junk) == 8


def test_reset_invalidates_tapes(fresh):
    from gorgonia_b200 import B200Error
    e = fresh
    a = e.tensor(np.ones(8, np.float32))
    e.Signal()
    e.tape_begin()
    e.AddScalar(a, 1.0, unsafe=True)
    with pytest.raises(B200Error) as ei:
        e.ResetAllocator()                               # refused while recording
    assert ei.value.code == 6
    t = e.tape_end()
    e.ResetAllocator()
    with pytest.raises(B200Error) as ei:
        e.tape_launch(t)
    assert ei.value.code == 6
    e.tape_destroy(t)


def test_recorded_gather_reports_bad_index_at_the_next_wait(fresh):
    from gorgonia_b200 import B200Error
    e = fresh
    x = e.tensor(util.normal(62, (10, 16)))
    idx = e.tensor(np.array([1, 3, 5], np.int64))
    y = e.tensor(np.zeros((3, 16), np.float32))
    e.Signal()
    e.tape_begin()
    e.ByIndices(x, idx, y)
    t = e.tape_end()
    e.tape_launch(t)
    assert_bits_equal(y.numpy(), x.numpy()[[1, 3, 5]])
    idx.set(np.array([1, 30, 5], np.int64))
    e.tape_launch(t)
    with pytest.raises(B200Error) as ei:
        e.Signal()
    assert ei.value.code == 1
    idx.set(np.array([0, 2, 4], np.int64))
    e.tape_launch(t)
    e.Signal()                                           # the error does not stick
    assert_bits_equal(y.numpy(), x.numpy()[[0, 2, 4]])
    e.tape_destroy(t)


def test_bounded_wait_that_runs_out_is_reported(fresh):
    # a warp waits 50 microseconds on a barrier nobody arrives at, gives up and returns; every entry
    # point that waits for the stream reports it, once, and the engine keeps working
    from gorgonia_b200 import B200Error, _lib
    e = fresh
    a = e.tensor(np.arange(8, dtype=np.float32))
    e.Signal()
    _lib.check(_lib.lib.b200_selftest_wait(e.h, 50), e.h)
    with pytest.raises(B200Error) as ei:
        e.Signal()
    assert ei.value.code == _lib.ERR_TIMEOUT
    e.Signal()
    _lib.check(_lib.lib.b200_selftest_wait(e.h, 50), e.h)
    with pytest.raises(B200Error) as ei:
        a.numpy()                                        # b200_memcpy_d2h
    assert ei.value.code == _lib.ERR_TIMEOUT
    _lib.check(_lib.lib.b200_selftest_wait(e.h, 50), e.h)
    with pytest.raises(B200Error) as ei:
        e.HasNaN(a)
    assert ei.value.code == _lib.ERR_TIMEOUT
    e.AddScalar(a, 1.0, unsafe=True)
    assert a.numpy().tolist() == [1, 2, 3, 4, 5, 6, 7, 8]


def test_tiny_yolo_with_weights_from_a_darknet_file(fresh, tmp_path):
    # weights travel file -> host fold -> device; the forward pass then matches the oracle run with the
    # same folded weights, also through the tape (recorded again by load_weights)
    from gorgonia_b200 import darknet
    e = fresh
    ch = (3, 16, 32, 64, 32, 64, 32, 64, 32, 20)
    m = tapes.TinyYolo(e, 2, size=64, channels=ch)
    x = util.uniform(140, (2, 3, 64, 64))
    m.x.set(x)
    m.record()
    g = util.rng(141)
    layers = []
    for i, shape in enumerate(darknet.layer_shapes(ch)):
        L = {"bias": (g.standard_normal(shape[0]) * 0.1).astype(np.float32),
             "kernel": (g.standard_normal(shape) * np.sqrt(2.0 / np.prod(shape[1:]))).astype(np.float32)}
        if i < 8:
            L.update(gamma=(1 + 0.1 * g.standard_normal(shape[0])).astype(np.float32),
                     mean=(0.1 * g.standard_normal(shape[0])).astype(np.float32),
                     var=(g.random(shape[0]) + 0.5).astype(np.float32))
        layers.append(L)
    path = str(tmp_path / "net.weights")
    darknet.write_tiny_yolo_v2(path, layers)
    m.load_weights(*darknet.load_tiny_yolo_v2(path, ch))
    got = m.forward().numpy()
    assert_gemm_close(got, graphs.tiny_yolo(m, x), 1e-5)
    m.replay()
    assert_bits_equal(m.out.numpy(), got)
    m.close()

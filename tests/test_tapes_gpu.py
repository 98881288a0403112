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

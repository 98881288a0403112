"""The three inference graphs evaluated op by op with the CPU oracle (TEST INFRASTRUCTURE ONLY).

Each function takes a tape object of gorgonia_b200.tapes (for its host copies of the weights) and
an input batch, and returns what gorgonia's CPU engine would: the same instruction sequence the
graphs of examples/286, examples/convnet and examples/tiny-yolo-v2-coco compile to.
"""
import numpy as np

from . import oracle


def mlp(m, x):
    a = x
    for i in range(3):
        a = oracle.gemm(a, m.w_host[i])
        a = oracle.binary_bcast("add", a, m.b_host[i], 1, a.shape[1])
        if i < 2:
            a = oracle.rectify(a)
    return oracle.softmax(a)


def lenet(m, x):
    a = x
    for i in range(3):
        a = oracle.rectify(oracle.conv2d(a, m.wc_host[i], (1, 1)))
        a, _ = oracle.maxpool2d(a, (2, 2), (0, 0), (2, 2))
    a = a.reshape(a.shape[0], 1152)
    a = oracle.rectify(oracle.gemm(a, m.wd_host[0]))
    return oracle.softmax(oracle.gemm(a, m.wd_host[1]))


def tiny_yolo(m, x):
    a = x
    for i in range(9):
        a = oracle.conv2d(a, m.w_host[i], (m.k[i] // 2,) * 2)
        a = (a + m.b_host[i][None, :, None, None]).astype(np.float32)
        a = oracle.leaky_relu(a, 1.0 if i == 8 else 0.1)
        if i < 5:
            a, _ = oracle.maxpool2d(a, (2, 2), (0, 0), (2, 2))
        elif i == 5:
            a, _ = oracle.maxpool2d(a, (2, 2), (1, 0, 1, 0), (1, 1))
    return a

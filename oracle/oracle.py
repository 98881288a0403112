"""numpy-facing wrapper of liboracle.so (oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the
CPU-baseline legs of bench.py. The product never imports it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

OP = {n: i for i, n in enumerate(["add", "sub", "mul", "div", "pow", "mod", "lt", "gt", "lte", "gte", "eq", "ne"])}
OP.update({n: 32 + i for i, n in enumerate(
    ["abs", "sign", "ceil", "floor", "sin", "cos", "exp", "ln", "log2", "neg", "square", "sqrt", "inv",
     "invsqrt", "cube", "tanh", "sigmoid", "log1p", "expm1", "softplus"])})


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE])


def _load():
    src = os.path.join(_HERE, "oracle.c")
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        build()
    return C.CDLL(_SO)


_lib = _load()
_i64 = C.c_int64
_vp = C.c_void_p


def _p(a):
    return a.ctypes.data_as(_vp)


def _sfx(dt):
    return {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64"}[np.dtype(dt)]


def threads():
    return int(_lib.oracle_threads())


def set_threads(n):
    """Number of OpenMP threads the oracle uses from now on (overrides OMP_NUM_THREADS)."""
    return int(_lib.oracle_set_threads(int(n)))


def binary(op, a, b):
    """a, b: arrays of the same shape, or 0-d / python scalars for the scalar operand."""
    a_s, b_s = np.ndim(a) == 0, np.ndim(b) == 0
    dt = (b if a_s else a).dtype
    a = np.ascontiguousarray(a, dtype=dt).reshape(-1) if not a_s else np.array([a], dtype=dt)
    shape = np.shape(b) if a_s else None
    bb = np.ascontiguousarray(b, dtype=dt).reshape(-1) if not b_s else np.array([b], dtype=dt)
    n = max(a.size, bb.size)
    out = np.empty(n, dtype=dt)
    getattr(_lib, "oracle_binary_" + _sfx(dt))(OP[op], _p(out), _p(a), _p(bb), _i64(n), int(a_s), int(b_s))
    return out


def unary(op, a):
    a = np.ascontiguousarray(a)
    out = np.empty_like(a)
    getattr(_lib, "oracle_unary_" + _sfx(a.dtype))(OP[op], _p(out), _p(a), _i64(a.size))
    return out


def binary_bcast(op, a, b, div, mod, bcast_is_a=False):
    full = b if bcast_is_a else a
    full = np.ascontiguousarray(full)
    a = np.ascontiguousarray(a, dtype=full.dtype)
    b = np.ascontiguousarray(b, dtype=full.dtype)
    out = np.empty(full.size, dtype=full.dtype)
    getattr(_lib, "oracle_binary_bcast_" + _sfx(full.dtype))(
        OP[op], _p(out), _p(a), _p(b), _i64(full.size), _i64(div), _i64(mod), int(bcast_is_a))
    return out.reshape(full.shape)


def gemm(A, B, transA=False, transB=False):
    A = np.ascontiguousarray(A)
    B = np.ascontiguousarray(B, dtype=A.dtype)
    M, K = (A.shape[1], A.shape[0]) if transA else A.shape
    N = B.shape[0] if transB else B.shape[1]
    Cm = np.empty((M, N), dtype=A.dtype)
    getattr(_lib, "oracle_gemm_" + _sfx(A.dtype))(int(transA), int(transB), _i64(M), _i64(N), _i64(K), _p(A),
                                                  _i64(A.shape[1]), _p(B), _i64(B.shape[1]), _p(Cm), _i64(N))
    return Cm


def gemm_f32_naive(A, B):
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    Cm = np.empty((A.shape[0], B.shape[1]), dtype=np.float32)
    _lib.oracle_gemm_f32_naive(_i64(A.shape[0]), _i64(B.shape[1]), _i64(A.shape[1]), _p(A), _p(B), _p(Cm))
    return Cm


def batched_matmul(A, B, transA=False, transB=False):
    """batchedMatMul (operatorLinAlg.go:435-502): equal leading dims, MatMul per slice."""
    lead = A.shape[:-2]
    A2 = A.reshape((-1,) + A.shape[-2:])
    B2 = B.reshape((-1,) + B.shape[-2:])
    outs = [gemm(A2[i], B2[i], transA, transB) for i in range(A2.shape[0])]
    return np.stack(outs).reshape(lead + outs[0].shape)


def gemv(A, x, transA=False):
    A = np.ascontiguousarray(A)
    x = np.ascontiguousarray(x, dtype=A.dtype)
    M, N = A.shape
    y = np.empty(N if transA else M, dtype=A.dtype)
    getattr(_lib, "oracle_gemv_" + _sfx(A.dtype))(int(transA), _i64(M), _i64(N), _p(A), _i64(N), _p(x), _p(y))
    return y


def outer(x, y):
    x = np.ascontiguousarray(x)
    y = np.ascontiguousarray(y, dtype=x.dtype)
    A = np.empty((x.size, y.size), dtype=x.dtype)
    getattr(_lib, "oracle_outer_" + _sfx(x.dtype))(_i64(x.size), _i64(y.size), _p(x), _p(y), _p(A))
    return A


def conv_out(h, k, pad, stride, dil=1):
    return (h + 2 * pad - (dil * (k - 1) + 1)) // stride + 1


def im2col(x, kh, kw, pad=(0, 0), stride=(1, 1), dil=(1, 1)):
    x = np.ascontiguousarray(x, dtype=np.float32)
    B, Cc, H, W = x.shape
    Ho, Wo = conv_out(H, kh, pad[0], stride[0], dil[0]), conv_out(W, kw, pad[1], stride[1], dil[1])
    col = np.empty((B, Ho, Wo, Cc * kh * kw), dtype=np.float32)
    _lib.oracle_im2col_f32(_p(x), _p(col), _i64(B), _i64(Cc), _i64(H), _i64(W), kh, kw, pad[0], pad[1], stride[0],
                           stride[1], dil[0], dil[1])
    return col


def conv2d(x, w, pad=(0, 0), stride=(1, 1), dil=(1, 1)):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    B, Cc, H, W = x.shape
    K, _, kh, kw = w.shape
    Ho, Wo = conv_out(H, kh, pad[0], stride[0], dil[0]), conv_out(W, kw, pad[1], stride[1], dil[1])
    y = np.empty((B, K, Ho, Wo), dtype=np.float32)
    _lib.oracle_conv2d_f32(_p(x), _p(w), _p(y), _i64(B), _i64(Cc), _i64(H), _i64(W), _i64(K), kh, kw, pad[0],
                           pad[1], stride[0], stride[1], dil[0], dil[1])
    return y


def maxpool2d(x, kernel, pad, stride):
    """pad: (ph, pw) symmetric, or (north, south, west, east) = gorgonia's explicit padding."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    B, Cc, H, W = x.shape
    if len(pad) == 2:
        pn, ps, pw, pe, explicit = pad[0], pad[0], pad[1], pad[1], 0
    else:
        pn, ps, pw, pe = pad
        explicit = 1
    Ho = (H + pn + ps - (kernel[0] - 1) - 1) // stride[0] + 1
    Wo = (W + pw + pe - (kernel[1] - 1) - 1) // stride[1] + 1
    y = np.empty((B, Cc, Ho, Wo), dtype=np.float32)
    mask = np.empty((B, Cc, Ho, Wo), dtype=np.int64)
    _lib.oracle_maxpool2d_f32(_p(x), _p(y), _p(mask), _i64(B), _i64(Cc), _i64(H), _i64(W), kernel[0], kernel[1],
                              pn, ps, pw, pe, explicit, stride[0], stride[1])
    return y, mask


def maxpool2d_bwd(dy, mask, in_shape):
    """Gradient of maxpool2d with respect to its input; mask as returned by maxpool2d."""
    dy = np.ascontiguousarray(dy)
    mask = np.ascontiguousarray(mask, dtype=np.int64)
    B, Cc, H, W = in_shape
    dx = np.empty(in_shape, dtype=dy.dtype)
    getattr(_lib, "oracle_maxpool2d_bwd_" + _sfx(dy.dtype))(_p(dy), _p(mask), _p(dx), _i64(B * Cc), _i64(H * W),
                                                            _i64(dy.shape[2] * dy.shape[3]))
    return dx


def col2im(col, in_shape, kh, kw, pad=(0, 0), stride=(1, 1), dil=(1, 1)):
    """col (B, Ho, Wo, C*kh*kw) accumulated back into an image of in_shape = (B, C, H, W)."""
    col = np.ascontiguousarray(col)
    B, Cc, H, W = in_shape
    im = np.empty(in_shape, dtype=col.dtype)
    getattr(_lib, "oracle_col2im_" + _sfx(col.dtype))(_p(col), _p(im), _i64(B), _i64(Cc), _i64(H), _i64(W), kh, kw,
                                                      pad[0], pad[1], stride[0], stride[1], dil[0], dil[1])
    return im


def softmax_bwd(y, grad, axis=-1, log=False):
    y = np.ascontiguousarray(y)
    grad = np.ascontiguousarray(grad, dtype=y.dtype)
    axis %= y.ndim
    o, l, i = _oli(y.shape, axis)
    dx = np.empty_like(y)
    getattr(_lib, "oracle_softmax_bwd_" + _sfx(y.dtype))(_p(y), _p(grad), _p(dx), _i64(o), _i64(l), _i64(i), int(log))
    return dx


def batchnorm(x, running_mean, running_var, training=True, momentum=0.9, eps=1e-5):
    """BatchNormOp on (B, C, ...) -> (y, save_mean, save_var); running_mean / running_var are
    updated in place when training."""
    x = np.ascontiguousarray(x)
    B, Cc = x.shape[0], x.shape[1]
    S = int(np.prod(x.shape[2:], dtype=np.int64)) if x.ndim > 2 else 1
    y = np.empty_like(x)
    sm, sv = np.zeros(Cc, x.dtype), np.zeros(Cc, x.dtype)
    assert running_mean.dtype == x.dtype and running_var.dtype == x.dtype
    getattr(_lib, "oracle_batchnorm_" + _sfx(x.dtype))(_p(x), _p(y), _i64(B), _i64(Cc), _i64(S), int(training),
                                                       C.c_double(momentum), C.c_double(eps), _p(running_mean),
                                                       _p(running_var), _p(sm), _p(sv))
    return y, sm, sv


def batchnorm_bwd(x, dy, running_var, save_mean, save_var, training=True, eps=1e-5):
    """batchnormDiffOp: the gradient with respect to the BatchNormOp input."""
    x = np.ascontiguousarray(x)
    dy = np.ascontiguousarray(dy, dtype=x.dtype)
    B, Cc = x.shape[0], x.shape[1]
    S = int(np.prod(x.shape[2:], dtype=np.int64)) if x.ndim > 2 else 1
    dx = np.empty_like(x)
    getattr(_lib, "oracle_batchnorm_bwd_" + _sfx(x.dtype))(_p(x), _p(dy), _p(dx), _i64(B), _i64(Cc), _i64(S),
                                                           int(training), C.c_double(eps), _p(running_var),
                                                           _p(save_mean), _p(save_var))
    return dx


def dropout(x, prob, uniforms=None, seed=0, offset=0):
    """dropoutOp in training mode: uniforms (same shape and dtype as x) or Philox keyed by seed."""
    x = np.ascontiguousarray(x)
    y = np.empty_like(x)
    u = None if uniforms is None else np.ascontiguousarray(uniforms, dtype=x.dtype)
    getattr(_lib, "oracle_dropout_" + _sfx(x.dtype))(_p(x), _p(y), _i64(x.size), C.c_double(prob),
                                                     _p(u) if u is not None else None, C.c_uint64(seed),
                                                     C.c_uint64(offset))
    return y


def dropout_bwd(dy, out, prob):
    dy = np.ascontiguousarray(dy)
    out = np.ascontiguousarray(out, dtype=dy.dtype)
    dx = np.empty_like(dy)
    getattr(_lib, "oracle_dropout_bwd_" + _sfx(dy.dtype))(_p(dy), _p(out), _p(dx), _i64(dy.size), C.c_double(prob))
    return dx


def _oli(shape, axis):
    outer_ = int(np.prod(shape[:axis], dtype=np.int64))
    inner = int(np.prod(shape[axis + 1:], dtype=np.int64))
    return outer_, shape[axis], inner


def softmax(x, axis=-1, log=False):
    x = np.ascontiguousarray(x)
    axis %= x.ndim
    o, l, i = _oli(x.shape, axis)
    y = np.empty_like(x)
    getattr(_lib, "oracle_softmax_" + _sfx(x.dtype))(_p(x), _p(y), _i64(o), _i64(l), _i64(i), int(log))
    return y


def reduce(kind, x, axis):
    x = np.ascontiguousarray(x)
    axis %= x.ndim
    o, l, i = _oli(x.shape, axis)
    y = np.empty(x.shape[:axis] + x.shape[axis + 1:], dtype=x.dtype)
    getattr(_lib, "oracle_reduce_" + _sfx(x.dtype))({"sum": 0, "max": 1}[kind], _p(x), _p(y), _i64(o), _i64(l),
                                                   _i64(i))
    return y


def argmax(x, axis):
    x = np.ascontiguousarray(x, dtype=np.float32)
    axis %= x.ndim
    o, l, i = _oli(x.shape, axis)
    y = np.empty(x.shape[:axis] + x.shape[axis + 1:], dtype=np.int64)
    _lib.oracle_argmax_f32(_p(x), _p(y), _i64(o), _i64(l), _i64(i))
    return y


def transpose(x, perm):
    x = np.ascontiguousarray(x)
    shape = (C.c_int64 * x.ndim)(*x.shape)
    pm = (C.c_int * x.ndim)(*perm)
    y = np.empty([x.shape[p] for p in perm], dtype=x.dtype)
    _lib.oracle_transpose(_p(x), _p(y), x.ndim, shape, pm, x.dtype.itemsize)
    return y


def gather_rows(x, idx):
    x = np.ascontiguousarray(x)
    idx = np.ascontiguousarray(idx, dtype=np.int64)
    row = int(np.prod(x.shape[1:], dtype=np.int64)) * x.dtype.itemsize
    y = np.empty((idx.size,) + x.shape[1:], dtype=x.dtype)
    _lib.oracle_gather_rows(_p(x), _p(idx), _p(y), _i64(idx.size), _i64(row))
    return y


def gather_axis(x, idx, axis):
    x = np.ascontiguousarray(x)
    idx = np.ascontiguousarray(idx, dtype=np.int64)
    axis %= x.ndim
    o, l, i = _oli(x.shape, axis)
    y = np.empty(x.shape[:axis] + (idx.size,) + x.shape[axis + 1:], dtype=x.dtype)
    _lib.oracle_gather_axis(_p(x), _p(idx), _p(y), _i64(o), _i64(l), _i64(idx.size), _i64(i * x.dtype.itemsize))
    return y


def rectify(x):
    """Rectify (nn.go:136-163): x * (x >= 0)."""
    return binary("mul", x.reshape(-1), binary("gte", x.reshape(-1), x.dtype.type(0))).reshape(x.shape)


def leaky_relu(x, alpha):
    """LeakyRelu (nn.go:83-131): x*(x>=0) + (x*(x<0))*alpha, in that association."""
    f = x.reshape(-1)
    z = x.dtype.type(0)
    pos = binary("mul", f, binary("gte", f, z))
    neg = binary("mul", binary("mul", f, binary("lt", f, z)), x.dtype.type(alpha))
    return binary("add", pos, neg).reshape(x.shape)

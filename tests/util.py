"""Shared helpers of the parity tests: seeded inputs and the tolerance definitions.

Tolerances (float32 unless stated):
  - compare ops, gather, argmax, masks: bit-exact;
  - pointwise: |g - r| <= 1e-6 * max(|r|, tiny) per element;
  - GEMM / conv: |g - r| <= 1e-5 * max(|r|, rms(r)) per element (1e-2 on the same scale for
    bf16 inputs); the rms floor is there because sums of zero-mean products land arbitrarily
    close to zero, where an element-wise relative error means nothing.
"""
import numpy as np

CMP_OPS = ("lt", "gt", "lte", "gte", "eq", "ne")
ARITH_OPS = ("add", "sub", "mul", "div", "pow", "mod")
UNARY_OPS = ("abs", "sign", "ceil", "floor", "sin", "cos", "exp", "ln", "log2", "neg", "square", "sqrt",
             "inv", "invsqrt", "cube", "tanh", "sigmoid", "log1p", "expm1", "softplus")
POSITIVE_DOMAIN = ("ln", "log2", "sqrt", "invsqrt", "log1p")
EDGE_SIZES = (1, 3, 4, 5, 31, 1023, 1024, 1025, 4099)
# above the size where the engine switches to its shared-memory-staged streaming kernel; not a
# multiple of the vector width, so the ragged tail is exercised too
STREAM_SIZE = (1 << 21) + 5


def rng(seed):
    return np.random.Generator(np.random.Philox(seed))


def normal(seed, shape, dtype=np.float32, scale=1.0):
    return (rng(seed).standard_normal(shape) * scale).astype(dtype)


def uniform(seed, shape, dtype=np.float32):
    return rng(seed).random(shape).astype(dtype)


def unary_input(op, seed, n, dtype=np.float32):
    x = normal(seed, n, dtype)
    if op in POSITIVE_DOMAIN:
        x = (np.abs(x) + dtype(0.1)).astype(dtype)
    return x


def assert_bits_equal(g, r):
    g = np.ascontiguousarray(g)
    r = np.ascontiguousarray(r)
    assert g.shape == r.shape and g.dtype == r.dtype
    u = {4: np.uint32, 8: np.uint64, 2: np.uint16}[g.dtype.itemsize]
    differ = g.view(u) != r.view(u)
    if g.dtype.kind == "f":
        # NaN has many encodings and IEEE 754 does not say which one an operation returns:
        # x86 and the GPU differ in sign and payload. Any NaN matches any NaN.
        differ &= ~(np.isnan(g) & np.isnan(r))
    bad = np.nonzero(differ)
    assert bad[0].size == 0, f"{bad[0].size} elements differ, first at {tuple(b[0] for b in bad)}"


def assert_pointwise_close(g, r, rel=None):
    g = np.asarray(g)
    r = np.asarray(r)
    assert g.shape == r.shape and g.dtype == r.dtype
    if rel is None:
        rel = 1e-6 if g.dtype == np.float32 else 1e-13
    tiny = np.finfo(g.dtype).tiny
    both_nan = np.isnan(g) & np.isnan(r)
    same_inf = np.isinf(r) & (g == r)
    with np.errstate(invalid="ignore"):
        err = np.abs(g.astype(np.float64) - r.astype(np.float64))
        lim = rel * np.maximum(np.abs(r.astype(np.float64)), tiny)
        ok = (err <= lim) | both_nan | same_inf
    if not ok.all():
        i = np.argmax(~ok)
        raise AssertionError(f"{(~ok).sum()} of {ok.size} elements off; first at {i}: got {g.flat[i]!r} want "
                             f"{r.flat[i]!r} (rel {err.flat[i] / max(abs(float(r.flat[i])), tiny):.3g})")


def assert_gemm_close(g, r, rel=1e-5):
    g = np.asarray(g, dtype=np.float64)
    r = np.asarray(r, dtype=np.float64)
    assert g.shape == r.shape
    rms = float(np.sqrt(np.mean(r * r))) if r.size else 0.0
    lim = rel * np.maximum(np.abs(r), rms)
    err = np.abs(g - r)
    ok = err <= lim
    if not ok.all():
        i = np.argmax(err / np.maximum(lim, 1e-300))
        raise AssertionError(f"{(~ok).sum()} of {ok.size} elements off; worst at {i}: got {g.flat[i]!r} want "
                             f"{r.flat[i]!r}, err {err.flat[i]:.3g} > {lim.flat[i]:.3g} (rms {rms:.3g})")

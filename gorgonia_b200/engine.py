"""Host-side mirror of gorgonia's `cuda.Engine` over the C ABI.

The method set, argument meaning and error behaviour follow gorgonia's cuda package
(cuda/engine.go:17-35 lists the interfaces it implements): Add/Sub/Mul/Div/Pow/Mod,
Lt/Lte/Gt/Gte/ElEq/ElNe with their *Scalar forms (cuda/arith.go, cuda/cmp.go),
MatMul/MatVecMul/Outer (cuda/linalg.go), Get/Put/ResetAllocator (cuda/arena.go),
HasNaN/HasInf (cuda/engine.go:144-191), Signal/DoWork/Sync (cuda/external.go:46-50,223-276).
The Go shim a gorgonia build would use calls the same C functions through cgo; this Python
class exists so the parity tests read like gorgonia's own tests.

Nothing here computes on the host: every method forwards to libgorgonia_b200.so.
"""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import B200Error, check, lib

_DT = {np.dtype(np.float32): _lib.F32, np.dtype(np.float64): _lib.F64}
BF16 = "bf16"  # dtype tag of bfloat16 tensors (held as uint16 on the host side)


def to_bf16(a):
    """float32 array -> bfloat16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


def from_bf16(u16):
    return (u16.astype(np.uint32) << 16).view(np.float32)


def _epilogue(bias=None, bias_kind=None, act=None, alpha=0.0, accumulate=False):
    if bias is None and act is None and not accumulate:
        return None
    ep = _lib.Epilogue()
    ep.bias_kind = 0 if bias is None else {"col": _lib.BIAS_COL, "row": _lib.BIAS_ROW}[bias_kind]
    ep.bias = None if bias is None else bias.ptr
    ep.act = {None: 0, "rectify": _lib.ACT_RECTIFY, "leaky": _lib.ACT_LEAKY}[act]
    ep.alpha = alpha
    ep.accumulate = 1 if accumulate else 0
    return ep


def dtype_code(dt):
    dt = np.dtype(dt)
    if dt not in _DT:
        raise B200Error(_lib.ERR_UNSUPPORTED, f"dtype {dt} not supported")
    return _DT[dt]


class Tensor:
    """A dense row-major tensor living in an engine's arena (the role `*tensor.Dense` with
    manually managed memory plays in gorgonia, values.go:129-148)."""

    def __init__(self, engine, ptr, shape, dtype, owned=True):
        self.engine = engine
        self.ptr = ptr
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self.owned = owned

    @property
    def size(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def nbytes(self):
        return self.size * self.dtype.itemsize

    def numpy(self):
        out = np.empty(self.shape, dtype=self.dtype)
        if out.size:
            check(lib.b200_memcpy_d2h(self.engine.h, out.ctypes.data, self.ptr, out.nbytes), self.engine.h)
        return out

    def set(self, arr):
        arr = np.ascontiguousarray(arr, dtype=self.dtype)
        assert arr.size == self.size
        if arr.size:
            check(lib.b200_memcpy_h2d(self.engine.h, self.ptr, arr.ctypes.data, arr.nbytes), self.engine.h)
        return self

    def reshape(self, *shape):
        t = Tensor(self.engine, self.ptr, shape, self.dtype, owned=False)
        assert t.size == self.size
        return t

    def free(self):
        if self.owned and self.ptr:
            self.engine.Put(self.ptr, self.nbytes)
            self.ptr = None


class Engine:
    def __init__(self, device=0, arena_bytes=1 << 30, managed=False, defer=True, conv_gather=False, streamk=True,
                 pairs=True):
        flags = ((_lib.ENGINE_MANAGED if managed else 0) | (0 if defer else _lib.ENGINE_NO_DEFER) |
                 (_lib.ENGINE_CONV_GATHER if conv_gather else 0) | (0 if streamk else _lib.ENGINE_NO_STREAMK) |
                 (0 if pairs else _lib.ENGINE_NO_PAIRS))
        h = C.c_void_p()
        rc = lib.b200_engine_create(device, arena_bytes, flags, C.byref(h))
        if rc != _lib.OK:
            raise B200Error(rc, (lib.b200_last_error(None) or b"").decode())
        self.h = h
        self.device = device

    # ---- lifecycle -------------------------------------------------------------------
    def Close(self):
        if self.h:
            lib.b200_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.Close()
        except Exception:
            pass

    def DoWork(self):
        check(lib.b200_flush(self.h), self.h)

    def Signal(self):
        check(lib.b200_sync(self.h), self.h)

    Sync = Signal

    @property
    def stream(self):
        return int(lib.b200_engine_stream(self.h))

    @property
    def launches(self):
        return int(lib.b200_launch_count(self.h))

    def pending(self):
        n, k = C.c_int(), C.c_int()
        check(lib.b200_pending(self.h, C.byref(n), C.byref(k)), self.h)
        return n.value, k.value

    # ---- tapes: record once, replay with one call ----------------------------------------
    def tape_begin(self):
        check(lib.b200_tape_begin(self.h), self.h)

    def tape_end(self):
        t = C.c_void_p()
        check(lib.b200_tape_end(self.h, C.byref(t)), self.h)
        return t

    def tape_launch(self, t):
        check(lib.b200_tape_launch(self.h, t), self.h)

    def tape_destroy(self, t):
        lib.b200_tape_destroy(self.h, t)

    def copy_h2d_async(self, t, host_ptr, nbytes=None):
        check(lib.b200_memcpy_h2d_async(self.h, t.ptr, host_ptr, t.nbytes if nbytes is None else nbytes), self.h)

    def upload_async(self, t, host_ptr, nbytes=None):
        """Host -> device on the engine's copy stream, overlapping compute queued after this call."""
        check(lib.b200_upload_async(self.h, t.ptr, host_ptr, t.nbytes if nbytes is None else nbytes), self.h)

    def upload_wait(self):
        check(lib.b200_upload_wait(self.h), self.h)

    def copy_d2h_async(self, host_ptr, t, nbytes=None):
        check(lib.b200_memcpy_d2h_async(self.h, host_ptr, t.ptr, t.nbytes if nbytes is None else nbytes), self.h)

    # ---- device timing -------------------------------------------------------------
    def event(self):
        ev = C.c_void_p()
        check(lib.b200_event_create(self.h, C.byref(ev)), self.h)
        return ev

    def record(self, ev):
        check(lib.b200_event_record(self.h, ev), self.h)

    def elapsed_ms(self, ev0, ev1):
        ms = C.c_float()
        check(lib.b200_event_elapsed_ms(self.h, ev0, ev1, C.byref(ms)), self.h)
        return ms.value

    def host_alloc(self, nbytes):
        p = C.c_void_p()
        rc = lib.b200_host_alloc(int(nbytes), C.byref(p))
        if rc != _lib.OK:
            raise B200Error(rc, (lib.b200_last_error(None) or b"").decode())
        return p.value

    # ---- arena -----------------------------------------------------------------------
    def Get(self, nbytes):
        p = C.c_void_p()
        check(lib.b200_get(self.h, int(nbytes), C.byref(p)), self.h)
        return p.value

    def Put(self, ptr, nbytes=0):
        check(lib.b200_put(self.h, ptr, int(nbytes)), self.h)

    def ResetAllocator(self):
        check(lib.b200_reset(self.h), self.h)

    def arena_stats(self):
        v = [C.c_int64() for _ in range(4)]
        check(lib.b200_arena_stats(self.h, *[C.byref(x) for x in v]), self.h)
        return dict(zip(("used", "free", "largest_free", "free_blocks"), (x.value for x in v)))

    # ---- tensors ---------------------------------------------------------------------
    def empty(self, shape, dtype=np.float32):
        if isinstance(shape, int):
            shape = (shape,)
        dtype = np.dtype(dtype)
        n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
        ptr = self.Get(max(n, 1) * dtype.itemsize)
        return Tensor(self, ptr, shape, dtype)

    def tensor(self, arr, dtype=None):
        arr = np.ascontiguousarray(arr, dtype=dtype)
        return self.empty(arr.shape, arr.dtype).set(arr)

    # ---- pointwise: Engine.<Op>(a, b, opts...) -----------------------------------------
    def _dest(self, a, reuse, unsafe, who):
        # cuda/arith.go:34-49: a reuse tensor, or unsafe; safe and incr are errors
        if reuse is not None:
            if reuse.size != a.size or reuse.dtype != a.dtype:
                raise B200Error(_lib.ERR_INVALID, f"{who}: reuse tensor does not match the operand")
            return reuse
        if unsafe:
            return a
        raise B200Error(_lib.ERR_INVALID,
                        f"{who}: a reuse tensor must be passed in, or the operation must be unsafe")

    def _binary(self, op, a, b, reuse=None, unsafe=False):
        if a.size != b.size or a.dtype != b.dtype:
            raise B200Error(_lib.ERR_INVALID, f"{op}: operands differ in size or dtype")
        dst = self._dest(a, reuse, unsafe, op)
        check(lib.b200_binary(self.h, _lib.OP[op], dtype_code(a.dtype), _lib.VV, dst.ptr, a.ptr, b.ptr, 0.0, 0,
                              a.size), self.h)
        return dst

    def _binary_scalar(self, op, t, s, leftTensor=True, reuse=None, unsafe=False):
        dst = self._dest(t, reuse, unsafe, op + "Scalar")
        on_dev = isinstance(s, Tensor)
        sval = 0.0 if on_dev else float(s)
        sptr = s.ptr if on_dev else None
        if leftTensor:
            rc = lib.b200_binary(self.h, _lib.OP[op], dtype_code(t.dtype), _lib.VS, dst.ptr, t.ptr, sptr, sval,
                                 int(on_dev), t.size)
        else:
            rc = lib.b200_binary(self.h, _lib.OP[op], dtype_code(t.dtype), _lib.SV, dst.ptr, sptr, t.ptr, sval,
                                 int(on_dev), t.size)
        check(rc, self.h)
        return dst

    def BroadcastBinary(self, op, a, b, div, mod, bcast_is_a=False, reuse=None, unsafe=False):
        full = b if bcast_is_a else a
        dst = self._dest(full, reuse, unsafe, op)
        check(lib.b200_binary_bcast(self.h, _lib.OP[op], dtype_code(full.dtype), dst.ptr, a.ptr, b.ptr, full.size,
                                    int(div), int(mod), int(bcast_is_a)), self.h)
        return dst

    def Unary(self, op, a, reuse=None, unsafe=False):
        dst = self._dest(a, reuse, unsafe, op)
        check(lib.b200_unary(self.h, _lib.OP[op], dtype_code(a.dtype), dst.ptr, a.ptr, a.size), self.h)
        return dst

    def BinaryIncr(self, op, a, b, incr):
        """Incr mode (execution.go:113-127): incr += op(a, b); a or b may be a python scalar."""
        a_s, b_s = not isinstance(a, Tensor), not isinstance(b, Tensor)
        t = b if a_s else a
        if incr.size != t.size or incr.dtype != t.dtype:
            raise B200Error(_lib.ERR_INVALID, f"{op}: incr tensor does not match the operand")
        form = _lib.SV if a_s else (_lib.VS if b_s else _lib.VV)
        check(lib.b200_binary_incr(self.h, _lib.OP[op], dtype_code(t.dtype), form, incr.ptr,
                                   None if a_s else a.ptr, None if b_s else b.ptr,
                                   float(a) if a_s else (float(b) if b_s else 0.0), 0, t.size), self.h)
        return incr

    def UnaryIncr(self, op, a, incr):
        check(lib.b200_unary_incr(self.h, _lib.OP[op], dtype_code(a.dtype), incr.ptr, a.ptr, a.size), self.h)
        return incr

    def Dropout(self, x, prealloc, prob, uniforms=None, seed=0, offset=0):
        """dropoutOp in training mode; `uniforms`: a tensor of draws in [0, 1), else Philox keyed by seed."""
        check(lib.b200_dropout_fwd(self.h, dtype_code(x.dtype), x.ptr, prealloc.ptr, x.size, float(prob),
                                   uniforms.ptr if uniforms is not None else None, int(seed), int(offset)), self.h)
        return prealloc

    def DropoutDiff(self, grad, out, prealloc, prob):
        check(lib.b200_dropout_bwd(self.h, dtype_code(grad.dtype), grad.ptr, out.ptr, prealloc.ptr, grad.size,
                                   float(prob)), self.h)
        return prealloc

    def Pointwise(self, prog, outs, srcs, n, dtype=np.float32):
        """prog: dict(instr=[(op, a_ref, b_ref)], imm=[...], out=[instr idx], bcast={src: (div, mod)})."""
        p = _lib.PwProg()
        p.n_instr = len(prog["instr"])
        p.n_src = len(srcs)
        p.n_imm = len(prog.get("imm", []))
        p.n_out = len(prog["out"])
        for k, (op, ra, rb) in enumerate(prog["instr"]):
            p.instr[k].op = _lib.OP[op]
            p.instr[k].a = ra
            p.instr[k].b = rb
        for k, v in enumerate(prog.get("imm", [])):
            p.imm[k] = v
        for k, v in enumerate(prog["out"]):
            p.out_instr[k] = v
        for s, (d, m) in prog.get("bcast", {}).items():
            p.src_div[s] = d
            p.src_mod[s] = m
        o = (C.c_void_p * len(outs))(*[t.ptr for t in outs])
        s = (C.c_void_p * max(len(srcs), 1))(*[t.ptr for t in srcs])
        check(lib.b200_pointwise(self.h, dtype_code(dtype), C.byref(p), o, s, int(n)), self.h)

    # ---- linear algebra: Engine.MatMul / MatVecMul / Outer (cuda/linalg.go) ---------------------
    def MatMul(self, a, b, prealloc, transA=False, transB=False, bias=None, bias_kind="col", act=None, alpha=0.0,
               incr=False):
        """prealloc = op(a) @ op(b), or prealloc += op(a) @ op(b) with incr (Incr mode, execution.go:115-126). a, b are 2-D (or N-D with equal leading dims: batched, as
        batchedMatMul, operatorLinAlg.go:435-502). bf16 operands (tensors made by tensor_bf16)
        give a float32 result."""
        bf = getattr(a, "is_bf16", False)
        if bf != getattr(b, "is_bf16", False):
            raise B200Error(_lib.ERR_INVALID, "MatMul: operand dtypes differ")
        if not bf and a.dtype != b.dtype:
            raise B200Error(_lib.ERR_INVALID, "MatMul: operand dtypes differ")
        if len(a.shape) != len(b.shape) or len(a.shape) < 2 or a.shape[:-2] != b.shape[:-2]:
            raise B200Error(_lib.ERR_INVALID, f"MatMul: shapes {a.shape} and {b.shape} do not match")
        batch = 1
        for d in a.shape[:-2]:
            batch *= d
        ar, ac = a.shape[-2:]
        br, bc = b.shape[-2:]
        M, K = (ac, ar) if transA else (ar, ac)
        K2, N = (bc, br) if transB else (br, bc)
        if K != K2:
            raise B200Error(_lib.ERR_INVALID, f"MatMul: inner dimensions differ ({K} vs {K2})")
        if prealloc.size != batch * M * N:
            raise B200Error(_lib.ERR_INVALID, "MatMul: prealloc has the wrong size")
        dt = _lib.BF16 if bf else dtype_code(a.dtype)
        ep = _epilogue(bias, bias_kind, act, alpha, accumulate=incr)
        check(lib.b200_gemm(self.h, dt, int(transA), int(transB), M, N, K, a.ptr, ac, b.ptr, bc, prealloc.ptr, N,
                            batch, ar * ac, br * bc, M * N, C.byref(ep) if ep else None), self.h)
        return prealloc

    def MatMulChain(self, a, b, c, M, N, K, transB=False, bias=None, bias_kind="col", act=None, alpha=0.0,
                    a_split=None, c_split=None, ld_split=0):
        """One link of a chain of dense layers. a / c: row-major tensors or None; a_split / c_split: (head, tail)
        pairs with row pitch K (rounded up to a multiple of 4 by the link that wrote them) / ld_split."""
        ep = _epilogue(bias, bias_kind, act, alpha)
        lda = a.shape[-1] if a is not None else a_split[0].shape[-1]
        check(lib.b200_gemm_chain(self.h, int(transB), M, N, K, a.ptr if a is not None else None,
                                  a_split[0].ptr if a_split else None, a_split[1].ptr if a_split else None, lda,
                                  b.ptr, b.shape[-1], c.ptr if c is not None else None,
                                  c_split[0].ptr if c_split else None, c_split[1].ptr if c_split else None,
                                  N, ld_split, C.byref(ep) if ep else None), self.h)

    def tf32_peak(self, batches=4096):
        """TFLOP/s of back-to-back kind::tf32 MMAs on every SM with no loads and no epilogue."""
        v = C.c_double()
        check(lib.b200_tf32_peak(self.h, int(batches), C.byref(v)), self.h)
        return v.value

    def gemm_path(self, a, b, c, transA=False, transB=False):
        bf = getattr(a, "is_bf16", False)
        ar, ac = a.shape[-2:]
        br, bc = b.shape[-2:]
        M, K = (ac, ar) if transA else (ar, ac)
        N = br if transB else bc
        return lib.b200_gemm_path(self.h, _lib.BF16 if bf else dtype_code(a.dtype), int(transA), int(transB), M, N, K,
                                  ac, bc, N, a.ptr, b.ptr, c.ptr)

    def MatVecMul(self, a, x, prealloc, transA=False):
        M, N = a.shape
        check(lib.b200_gemv(self.h, dtype_code(a.dtype), int(transA), M, N, a.ptr, N, x.ptr, prealloc.ptr), self.h)
        return prealloc

    def Outer(self, x, y, prealloc):
        check(lib.b200_ger(self.h, dtype_code(x.dtype), x.size, y.size, x.ptr, y.ptr, prealloc.ptr), self.h)
        return prealloc

    def constant(self, t, flag=True):
        """Declares a tensor constant (weights): what the engine derives from it is kept across calls."""
        check(lib.b200_set_constant(self.h, t.ptr, int(flag)), self.h)
        return t

    def tensor_bf16(self, arr):
        """Uploads a float32 array rounded to bfloat16."""
        u = to_bf16(arr)
        t = self.empty(u.shape, np.uint16).set(u)
        t.is_bf16 = True
        return t

    # ---- softmax / reductions ---------------------------------------------------------------
    @staticmethod
    def _oli(shape, axis):
        axis %= len(shape)
        o = int(np.prod(shape[:axis], dtype=np.int64))
        i = int(np.prod(shape[axis + 1:], dtype=np.int64))
        return o, shape[axis], i, axis

    def SoftMax(self, x, prealloc, axis=-1, log=False):
        o, l, i, _ = self._oli(x.shape, axis)
        check(lib.b200_softmax(self.h, dtype_code(x.dtype), x.ptr, prealloc.ptr, o, l, i, int(log)), self.h)
        return prealloc

    def SoftMaxDiff(self, y, grad, prealloc, axis=-1, log=False):
        """softmaxDiffOp: the gradient with respect to the softmax input, from its output y and dL/dy."""
        o, l, i, _ = self._oli(y.shape, axis)
        check(lib.b200_softmax_bwd(self.h, dtype_code(y.dtype), y.ptr, grad.ptr, prealloc.ptr, o, l, i, int(log)),
              self.h)
        return prealloc

    def Reduce(self, kind, x, prealloc, axis):
        o, l, i, _ = self._oli(x.shape, axis)
        check(lib.b200_reduce(self.h, dtype_code(x.dtype), {"sum": 0, "max": 1}[kind], x.ptr, prealloc.ptr, o, l, i),
              self.h)
        return prealloc

    def ReduceAll(self, kind, x, prealloc):
        check(lib.b200_reduce_all(self.h, dtype_code(x.dtype), {"sum": 0, "max": 1}[kind], x.ptr, x.size,
                                  prealloc.ptr), self.h)
        return prealloc

    def Argmax(self, x, prealloc, axis):
        o, l, i, _ = self._oli(x.shape, axis)
        check(lib.b200_argmax(self.h, dtype_code(x.dtype), x.ptr, prealloc.ptr, o, l, i), self.h)
        return prealloc

    # ---- nn -----------------------------------------------------------------------------------
    def Conv2d(self, x, w, prealloc, pad=(0, 0), stride=(1, 1), dil=(1, 1), bias=None, act=None, alpha=0.0):
        B, Cc, H, W = x.shape
        K, _, kh, kw = w.shape
        ep = _epilogue(bias, "row", act, alpha)
        check(lib.b200_conv2d_fwd(self.h, dtype_code(x.dtype), x.ptr, w.ptr, prealloc.ptr, B, Cc, H, W, K, kh, kw,
                                  pad[0], pad[1], stride[0], stride[1], dil[0], dil[1],
                                  C.byref(ep) if ep else None), self.h)
        return prealloc

    def Conv2dMaxPool(self, x, w, prealloc, pad=(0, 0), stride=(1, 1), dil=(1, 1), bias=None, act=None, alpha=0.0,
                      pool=(2, 2), pool_stride=(2, 2)):
        """Conv2d -> bias -> activation -> MaxPool2D (no pool padding) as one call; prealloc is the pooled output."""
        B, Cc, H, W = x.shape
        K, _, kh, kw = w.shape
        ep = _epilogue(bias, "row", act, alpha)
        check(lib.b200_conv2d_maxpool_fwd(self.h, dtype_code(x.dtype), x.ptr, w.ptr, prealloc.ptr, B, Cc, H, W, K, kh,
                                          kw, pad[0], pad[1], stride[0], stride[1], dil[0], dil[1],
                                          C.byref(ep) if ep else None, pool[0], pool[1], pool_stride[0],
                                          pool_stride[1]), self.h)
        return prealloc

    def Conv2dChain(self, x, w, y, in_shape, pad=(0, 0), stride=(1, 1), dil=(1, 1), bias=None, act=None, alpha=0.0,
                    pool2=False, x_split=None, y_split=None):
        """One link of a chain of convolutions. x / y: NCHW tensors or None; x_split / y_split: (head, tail)
        tensor pairs in NHWC TF32-split form or None; in_shape = (B, C, H, W) of the input."""
        B, Cc, H, W = in_shape
        K, _, kh, kw = w.shape
        ep = _epilogue(bias, "row", act, alpha)
        check(lib.b200_conv2d_chain_fwd(self.h, x.ptr if x is not None else None,
                                        x_split[0].ptr if x_split else None, x_split[1].ptr if x_split else None,
                                        w.ptr, y.ptr if y is not None else None,
                                        y_split[0].ptr if y_split else None, y_split[1].ptr if y_split else None,
                                        B, Cc, H, W, K, kh, kw, pad[0], pad[1], stride[0], stride[1], dil[0], dil[1],
                                        C.byref(ep) if ep else None, int(pool2)), self.h)

    def conv2d_path(self, x, w, pad=(0, 0), stride=(1, 1), dil=(1, 1)):
        """Which kernel Conv2d would run for these operands (one of the _lib.CONV_* values)."""
        B, Cc, H, W = x.shape
        K, _, kh, kw = w.shape
        return lib.b200_conv2d_path(self.h, dtype_code(x.dtype), B, Cc, H, W, K, kh, kw, pad[0], pad[1], stride[0],
                                    stride[1], dil[0], dil[1])

    def Im2Col(self, x, prealloc, kernel, pad=(0, 0), stride=(1, 1), dil=(1, 1)):
        B, Cc, H, W = x.shape
        check(lib.b200_im2col(self.h, dtype_code(x.dtype), x.ptr, prealloc.ptr, B, Cc, H, W, kernel[0], kernel[1],
                              pad[0], pad[1], stride[0], stride[1], dil[0], dil[1]), self.h)
        return prealloc

    def MaxPool2D(self, x, prealloc, kernel, pad, stride, mask=None):
        """pad: (ph, pw), or (north, south, west, east) = gorgonia's explicit padding."""
        B, Cc, H, W = x.shape
        if len(pad) == 2:
            pn, ps, pw, pe, explicit = pad[0], pad[0], pad[1], pad[1], 0
        else:
            pn, ps, pw, pe = pad
            explicit = 1
        check(lib.b200_maxpool2d_fwd(self.h, dtype_code(x.dtype), x.ptr, prealloc.ptr, mask.ptr if mask else None,
                                     B, Cc, H, W, kernel[0], kernel[1], pn, ps, pw, pe, explicit, stride[0],
                                     stride[1]), self.h)
        return prealloc

    def MaxPool2DSplit(self, x, prealloc, split, kernel, pad, stride):
        """MaxPool2D whose result goes to a convolution chain: split = (head, tail) NHWC tensors; prealloc
        (NCHW) may be None."""
        B, Cc, H, W = x.shape
        if len(pad) == 2:
            pn, ps, pw, pe, explicit = pad[0], pad[0], pad[1], pad[1], 0
        else:
            pn, ps, pw, pe = pad
            explicit = 1
        check(lib.b200_maxpool2d_split_fwd(self.h, x.ptr, prealloc.ptr if prealloc is not None else None,
                                           split[0].ptr, split[1].ptr, B, Cc, H, W, kernel[0], kernel[1], pn, ps, pw,
                                           pe, explicit, stride[0], stride[1]), self.h)
        return split

    def BatchNorm(self, x, prealloc, running_mean, running_var, save_mean=None, save_var=None, training=True,
                  momentum=0.9, epsilon=1e-5):
        """BatchNormOp on (B, C, ...): normalisation only; scale and bias are separate broadcast ops."""
        B, Cc = x.shape[0], x.shape[1]
        S = 1
        for d in x.shape[2:]:
            S *= d
        check(lib.b200_batchnorm_fwd(self.h, dtype_code(x.dtype), x.ptr, prealloc.ptr, B, Cc, S, int(training),
                                     momentum, epsilon, running_mean.ptr, running_var.ptr,
                                     save_mean.ptr if save_mean else None, save_var.ptr if save_var else None), self.h)
        return prealloc

    def BatchNormDiff(self, x, grad, prealloc, running_var, save_mean, save_var, training=True, epsilon=1e-5):
        """batchnormDiffOp: the gradient with respect to the BatchNorm input."""
        B, Cc = x.shape[0], x.shape[1]
        S = 1
        for d in x.shape[2:]:
            S *= d
        check(lib.b200_batchnorm_bwd(self.h, dtype_code(x.dtype), x.ptr, grad.ptr, prealloc.ptr, B, Cc, S,
                                     int(training), epsilon, running_var.ptr, save_mean.ptr, save_var.ptr), self.h)
        return prealloc

    def MaxPool2DDiff(self, grad, mask, prealloc, kernel, pad, stride):
        """maxPoolDiffOp: prealloc (B,C,H,W) = gradient of the pool input; mask as MaxPool2D wrote it."""
        B, Cc, H, W = prealloc.shape
        if len(pad) == 2:
            pn, ps, pw, pe, explicit = pad[0], pad[0], pad[1], pad[1], 0
        else:
            pn, ps, pw, pe = pad
            explicit = 1
        check(lib.b200_maxpool2d_bwd(self.h, dtype_code(grad.dtype), grad.ptr, mask.ptr, prealloc.ptr, B, Cc, H, W,
                                     kernel[0], kernel[1], pn, ps, pw, pe, explicit, stride[0], stride[1]), self.h)
        return prealloc

    def Col2Im(self, col, prealloc, kernel, pad=(0, 0), stride=(1, 1), dil=(1, 1)):
        """col2imOp: col (B, Ho, Wo, C*kh*kw) accumulated into prealloc (B,C,H,W)."""
        B, Cc, H, W = prealloc.shape
        check(lib.b200_col2im(self.h, dtype_code(col.dtype), col.ptr, prealloc.ptr, B, Cc, H, W, kernel[0], kernel[1],
                              pad[0], pad[1], stride[0], stride[1], dil[0], dil[1]), self.h)
        return prealloc

    def Transpose(self, x, prealloc, perm):
        shape = (C.c_int64 * len(x.shape))(*x.shape)
        pm = (C.c_int * len(perm))(*perm)
        check(lib.b200_transpose(self.h, x.dtype.itemsize, x.ptr, prealloc.ptr, len(x.shape), shape, pm), self.h)
        return prealloc

    def ByIndices(self, x, idx, prealloc, axis=0):
        outer, n_rows, inner, _ = self._oli(x.shape, axis)
        check(lib.b200_gather_axis(self.h, x.ptr, idx.ptr, prealloc.ptr, outer, n_rows, idx.size,
                                   inner * x.dtype.itemsize), self.h)
        return prealloc

    def HasNaN(self, t):
        r = C.c_int()
        check(lib.b200_has_nan(self.h, dtype_code(t.dtype), t.ptr, t.size, C.byref(r)), self.h)
        return bool(r.value)

    def HasInf(self, t):
        r = C.c_int()
        check(lib.b200_has_inf(self.h, dtype_code(t.dtype), t.ptr, t.size, C.byref(r)), self.h)
        return bool(r.value)


def _mk(op, name):
    def f(self, a, b, reuse=None, unsafe=False):
        return self._binary(op, a, b, reuse, unsafe)

    def fs(self, t, s, leftTensor=True, reuse=None, unsafe=False):
        return self._binary_scalar(op, t, s, leftTensor, reuse, unsafe)

    f.__name__ = name
    fs.__name__ = name + "Scalar"
    setattr(Engine, name, f)
    setattr(Engine, name + "Scalar", fs)


for _op, _name in [("add", "Add"), ("sub", "Sub"), ("mul", "Mul"), ("div", "Div"), ("pow", "Pow"),
                   ("mod", "Mod"), ("lt", "Lt"), ("lte", "Lte"), ("gt", "Gt"), ("gte", "Gte"),
                   ("eq", "ElEq"), ("ne", "ElNe")]:
    _mk(_op, _name)

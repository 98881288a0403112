"""Forward tapes of gorgonia's three inference graphs, issued as engine calls.

What the Go tape machine would do instruction by instruction (execOp.exec, vm_tape_cuda.go:66-150)
is spelled out here as the same sequence of engine calls, so that the parity tests and the
benchmark drive the library the way a gorgonia build would:

  MLP      examples/286/main.go:72-99 extended to 784-300-100-10 with biases: Mul -> BroadcastAdd ->
           Rectify, twice; Mul -> BroadcastAdd -> SoftMax.
  LeNet    examples/convnet/main.go:83-159 without the dropouts: (Conv2d 3x3 pad 1 -> Rectify ->
           MaxPool2D 2x2) x3, Reshape, Mul -> Rectify, Mul -> SoftMax.
  TinyYOLO examples/tiny-yolo-v2-coco/feedforward.go:46-187 with batch-norm folded: 9 x (Conv2d ->
           Add bias -> LeakyRelu), 2x2/2 pools after the first five, a 2x2/1 pool with gorgonia's
           explicit padding {1,0,1,0} after the sixth.

Every class owns its device buffers (weights stay resident across runs, unlike the reference,
which re-uploads them after each Reset: vm_tape.go:123-134, analysis.go:151-176), exposes
forward() = one pass of engine calls, and record()/replay() = the same pass as one recorded tape.
`fused=True` uses the fused bias/activation stores of b200_gemm and runs the convolutions as links
of b200_conv2d_chain_fwd: a 2x2/2 pool that follows a convolution is folded into it (the
convolution output is then never materialised) and a tensor that only the next convolution reads
is written directly in the layout that convolution's kernel reads; `fused=False` issues one
engine call per reference instruction and leaves fusing to the engine's deferred queue.
Weights are seeded draws (Glorot-uniform / He-normal formulas of weights.go:397-479); nothing is
computed on the host.
"""
import numpy as np


def _rng(seed):
    return np.random.Generator(np.random.Philox(seed))


def glorot_uniform(g, shape):
    """weights.go:397-427: U(-a, a), a = sqrt(3) * sqrt(2 / ((n1 + n2) * field)), gain 1."""
    field = int(np.prod(shape[2:])) if len(shape) > 2 else 1
    a = np.sqrt(3.0) * np.sqrt(2.0 / ((shape[0] + shape[1]) * field))
    return ((g.random(shape) * 2 - 1) * a).astype(np.float32)


def he_normal(g, shape, fan_in):
    """weights.go:455-479: N(0, sigma), sigma = sqrt(2) * sqrt(1 / fan_in)."""
    return (g.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)


class _Tape:
    def __init__(self, engine):
        self.e = engine
        self.tape = None

    def record(self):
        """Runs forward() once for set-up, then records it; replay() re-runs it with one call."""
        self.forward()
        self.e.Signal()
        self.e.tape_begin()
        self.forward()
        self.tape = self.e.tape_end()
        return self

    def replay(self):
        self.e.tape_launch(self.tape)

    def close(self):
        if self.tape is not None:
            self.e.tape_destroy(self.tape)
            self.tape = None


class _ConvChain:
    """Plans a run of convolutions (each optionally followed by a 2x2/2 max-pool) as links of
    b200_conv2d_chain_fwd: which links fold their pool in, and which tensors between links exist in
    NCHW, in the NHWC TF32-split form the tensor-core kernels read, or both."""

    def __init__(self, engine, batch, in_shape, layers):
        # layers: dicts with w, pad, bias, act, alpha, pool ('2x2/2' | None)
        from . import _lib
        e = engine
        self.e, self.layers = e, layers
        shape = (batch,) + tuple(in_shape)
        split_paths = (_lib.CONV_TC_WINDOW, _lib.CONV_TC_TMA)
        for L in layers:
            K, _, kh, kw = L["w"].shape
            B, Cc, H, W = shape
            Ho, Wo = H + 2 * L["pad"][0] - (kh - 1), W + 2 * L["pad"][1] - (kw - 1)
            L["in_shape"] = shape
            L["path"] = e.conv2d_path(_Shape(shape), L["w"], L["pad"])
            even = Ho % 2 == 0 and Wo % 2 == 0
            first = L["path"] == _lib.CONV_DIRECT and Cc <= 3 and kh == 3 and kw == 3 and L["pad"] == (1, 1) and W % 4 == 0
            L["fuse_pool"] = bool(L["pool"]) and even and (L["path"] == _lib.CONV_TC_WINDOW or first)
            L["conv_shape"] = (B, K, Ho, Wo)
            shape = (B, K, Ho // 2, Wo // 2) if L["pool"] else (B, K, Ho, Wo)
            L["out_shape"] = shape
        for i, L in enumerate(layers):
            nxt = layers[i + 1] if i + 1 < len(layers) else None
            direct_feed = not L["pool"] or L["fuse_pool"]       # the link's own output is what the next conv reads
            L["want_split"] = bool(nxt) and nxt["path"] in split_paths and direct_feed and L["w"].shape[0] % 4 == 0
            # NCHW is needed by a separate pool, by a next link whose kernel reads NCHW, and at the end
            L["want_nchw"] = not L["want_split"] or not direct_feed or nxt is None
        for i, L in enumerate(layers):
            nxt = layers[i + 1] if i + 1 < len(layers) else None
            B, K, Ho, Wo = L["conv_shape"]
            ob = L["out_shape"]
            sep_pool = bool(L["pool"]) and not L["fuse_pool"]
            L["y"] = e.empty(L["conv_shape"] if sep_pool else ob) if L["want_nchw"] else None
            L["split"] = (e.empty((ob[0], ob[2], ob[3], ob[1])), e.empty((ob[0], ob[2], ob[3], ob[1]))) \
                if L["want_split"] else None
            # a separate pool in front of a kernel that reads the split form writes that form itself
            L["pool_split"] = None
            if sep_pool and nxt is not None and nxt["path"] in split_paths:
                L["pool_split"] = (e.empty((ob[0], ob[2], ob[3], ob[1])), e.empty((ob[0], ob[2], ob[3], ob[1])))
            L["pooled"] = e.empty(ob) if (sep_pool and L["pool_split"] is None) else None

    def forward(self, x, x_split=None):
        e, a, a_split = self.e, x, x_split
        for L in self.layers:
            e.Conv2dChain(a, L["w"], L["y"], L["in_shape"], pad=L["pad"], bias=L["bias"], act=L["act"], alpha=L["alpha"],
                          pool2=L["fuse_pool"], x_split=a_split, y_split=L["split"])
            a, a_split = L["y"], L["split"]
            if L["pool_split"] is not None:
                a_split = e.MaxPool2DSplit(L["y"], None, L["pool_split"], (2, 2), (0, 0), (2, 2))
                a = None
            elif L["pooled"] is not None:
                e.MaxPool2D(L["y"], L["pooled"], (2, 2), (0, 0), (2, 2))
                a = L["pooled"]
        return a

    @property
    def reads_split(self):
        """Whether the first link's kernel reads the NHWC TF32-split form."""
        from . import _lib
        return self.layers[0]["path"] in (_lib.CONV_TC_WINDOW, _lib.CONV_TC_TMA)


class _DenseChain:
    """Plans a stack of dense layers act(a @ W + b) as links of b200_gemm_chain: an activation that
    only the next tensor-core product reads is written split into TF32 head and tail by the link
    that makes it, and never in plain form."""

    def __init__(self, engine, batch, layers):
        # layers: dicts with w (K, N), bias, act; the last layer's plain output is always kept
        e = engine
        self.e, self.batch, self.layers = e, batch, layers
        for L in layers:
            K, N = L["w"].shape
            probe_a, probe_c = _Shape((batch, K)), _Shape((batch, N))
            probe_a.ptr = probe_c.ptr = L["w"].ptr       # only alignment is looked at
            L["tc"] = e.gemm_path(probe_a, L["w"], probe_c) == 1
        for i, L in enumerate(layers):
            nxt = layers[i + 1] if i + 1 < len(layers) else None
            K, N = L["w"].shape
            L["want_split"] = L["tc"] and nxt is not None and nxt["tc"]
            L["pitch"] = (N + 3) // 4 * 4
            L["c"] = None if L["want_split"] else e.empty((batch, N))
            L["split"] = (e.empty((batch, L["pitch"])), e.empty((batch, L["pitch"]))) if L["want_split"] else None

    def forward(self, a):
        e, a_split = self.e, None
        for L in self.layers:
            K, N = L["w"].shape
            e.MatMulChain(a, L["w"], L["c"], self.batch, N, K, bias=L["bias"], bias_kind="col", act=L["act"],
                          a_split=a_split, c_split=L["split"], ld_split=L["pitch"] if L["split"] else 0)
            a, a_split = L["c"], L["split"]
        return a


class _Shape:
    """Stands in for a tensor where only shape and dtype are asked for."""

    def __init__(self, shape):
        self.shape, self.dtype = shape, np.dtype(np.float32)


class MLP(_Tape):
    DIMS = (784, 300, 100, 10)

    def __init__(self, engine, batch, seed=286, fused=True):
        super().__init__(engine)
        e, g = engine, _rng(seed)
        self.batch, self.fused = batch, fused
        self.w_host = [glorot_uniform(g, (self.DIMS[i], self.DIMS[i + 1])) for i in range(3)]
        self.b_host = [np.zeros(self.DIMS[i + 1], np.float32) for i in range(3)]
        self.w = [e.constant(e.tensor(w)) for w in self.w_host]
        self.b = [e.tensor(b) for b in self.b_host]
        self.x = e.empty((batch, 784))
        self.h = [e.empty((batch, d)) for d in self.DIMS[1:]]
        self.mask = [e.empty((batch, d)) for d in self.DIMS[1:3]]
        self.out = e.empty((batch, 10))
        self.chain = _DenseChain(e, batch, [
            {"w": self.w[i], "bias": self.b[i], "act": None if i == 2 else "rectify"} for i in range(3)]) if fused else None

    def forward(self):
        e, a = self.e, self.x
        if self.fused:
            e.SoftMax(self.chain.forward(a), self.out)
            return self.out
        for i in range(3):
            e.MatMul(a, self.w[i], self.h[i])
            e.BroadcastBinary("add", self.h[i], self.b[i], 1, self.DIMS[i + 1], unsafe=True)
            if i < 2:   # Rectify (nn.go:154-162): gte(x, 0) as float, then mul
                e.GteScalar(self.h[i], 0.0, reuse=self.mask[i])
                e.Mul(self.h[i], self.mask[i], unsafe=True)
            a = self.h[i]
        e.SoftMax(a, self.out)
        return self.out

    @property
    def flops_per_sample(self):
        return 2 * sum(self.DIMS[i] * self.DIMS[i + 1] for i in range(3))


class LeNet(_Tape):
    CH = (1, 32, 64, 128)

    def __init__(self, engine, batch, seed=5, fused=True):
        super().__init__(engine)
        e, g = engine, _rng(seed)
        self.batch, self.fused = batch, fused
        self.wc_host = [he_normal(g, (self.CH[i + 1], self.CH[i], 3, 3), self.CH[i] * 9) for i in range(3)]
        self.wd_host = [he_normal(g, (1152, 625), 1152), he_normal(g, (625, 10), 625)]
        self.wc = [e.constant(e.tensor(w)) for w in self.wc_host]
        self.wd = [e.constant(e.tensor(w)) for w in self.wd_host]
        self.x = e.empty((batch, 1, 28, 28))
        hw = (28, 14, 7)
        self.conv = [None if fused else e.empty((batch, self.CH[i + 1], hw[i], hw[i])) for i in range(3)]
        self.cmask = [None if fused else e.empty((batch, self.CH[i + 1], hw[i], hw[i])) for i in range(3)]
        self.pool = [None if fused else e.empty((batch, self.CH[i + 1], hw[i] // 2, hw[i] // 2)) for i in range(3)]
        self.chain = _ConvChain(e, batch, (1, 28, 28), [
            {"w": self.wc[i], "pad": (1, 1), "bias": None, "act": "rectify", "alpha": 0.0, "pool": "2x2/2"}
            for i in range(3)]) if fused else None
        self.dense = _DenseChain(e, batch, [{"w": self.wd[0], "bias": None, "act": "rectify"},
                                            {"w": self.wd[1], "bias": None, "act": None}]) if fused else None
        self.fc = e.empty((batch, 625))
        self.fmask = None if fused else e.empty((batch, 625))
        self.logits = e.empty((batch, 10))
        self.out = e.empty((batch, 10))

    def forward(self):
        e, a = self.e, self.x
        if self.fused:
            a = self.chain.forward(a)
        else:
            for i in range(3):
                e.Conv2d(a, self.wc[i], self.conv[i], pad=(1, 1))
                e.GteScalar(self.conv[i], 0.0, reuse=self.cmask[i])
                e.Mul(self.conv[i], self.cmask[i], unsafe=True)
                e.MaxPool2D(self.conv[i], self.pool[i], (2, 2), (0, 0), (2, 2))
                a = self.pool[i]
        flat = a.reshape(self.batch, 1152)
        if self.fused:
            e.SoftMax(self.dense.forward(flat), self.out)
            return self.out
        e.MatMul(flat, self.wd[0], self.fc)
        e.GteScalar(self.fc, 0.0, reuse=self.fmask)
        e.Mul(self.fc, self.fmask, unsafe=True)
        e.MatMul(self.fc, self.wd[1], self.logits)
        e.SoftMax(self.logits, self.out)
        return self.out

    @property
    def flops_per_sample(self):
        conv = 2 * (28 * 28 * 32 * 9 + 14 * 14 * 64 * 288 + 7 * 7 * 128 * 576)
        return conv + 2 * (1152 * 625 + 625 * 10)


class TinyYolo(_Tape):
    CH = (3, 16, 32, 64, 128, 256, 512, 1024, 1024, 125)

    def __init__(self, engine, batch, seed=9, size=416, channels=None, fused=True):
        super().__init__(engine)
        e, g = engine, _rng(seed)
        ch = tuple(channels) if channels else self.CH
        self.ch, self.batch, self.size, self.fused = ch, batch, size, fused
        self.k = [3] * 8 + [1]
        self.w_host = [he_normal(g, (ch[i + 1], ch[i], self.k[i], self.k[i]), ch[i] * self.k[i] ** 2)
                       for i in range(9)]
        self.b_host = [(g.standard_normal(ch[i + 1]) * 0.1).astype(np.float32) for i in range(9)]
        self.w = [e.constant(e.tensor(w)) for w in self.w_host]
        self.b = [e.tensor(b) for b in self.b_host]
        self.x = e.empty((batch, 3, size, size))
        s = size
        self.conv, self.pool = [], []
        for i in range(9):
            self.conv.append(None if fused else e.empty((batch, ch[i + 1], s, s)))
            if i < 5:
                s //= 2
                self.pool.append(None if fused else e.empty((batch, ch[i + 1], s, s)))
            elif i == 5:
                self.pool.append(e.empty((batch, ch[i + 1], s, s)))
        self.pool5_split = None
        if fused:
            def layer(i):
                return {"w": self.w[i], "pad": (self.k[i] // 2, self.k[i] // 2), "bias": self.b[i], "act": "leaky",
                        "alpha": 1.0 if i == 8 else 0.1, "pool": "2x2/2" if i < 5 else None}
            # two runs of links, cut by the 2x2 / stride-1 pool with explicit padding after layer 5
            self.chain_a = _ConvChain(e, batch, (3, size, size), [layer(i) for i in range(6)])
            self.chain_b = _ConvChain(e, batch, (ch[6], s, s), [layer(i) for i in range(6, 9)])
            if self.chain_b.reads_split:
                self.pool5_split = (e.empty((batch, s, s, ch[6])), e.empty((batch, s, s, ch[6])))
            self.out = self.chain_b.layers[-1]["y"]
        else:
            self.out = self.conv[8]

    def load_weights(self, kernels, biases):
        """Replaces the seeded weights, e.g. by what darknet.load_tiny_yolo_v2 read from a file. What the
        engine derived from the old values is dropped by withdrawing and renewing the constant
        declaration; a tape recorded earlier reads those derived forms, so it is recorded again."""
        e = self.e
        e.Signal()
        had_tape = self.tape is not None
        self.close()
        for i in range(9):
            w, b = np.ascontiguousarray(kernels[i], np.float32), np.ascontiguousarray(biases[i], np.float32)
            if w.shape != self.w[i].shape or b.shape != self.b[i].shape:
                raise ValueError(f"layer {i}: got {w.shape} / {b.shape}, the tape has {self.w[i].shape} / {self.b[i].shape}")
            e.constant(self.w[i], False)
            self.w[i].set(w)
            self.b[i].set(b)
            e.constant(self.w[i])
            self.w_host[i], self.b_host[i] = w, b
        if had_tape:
            self.record()
        return self

    def forward(self):
        e, a = self.e, self.x
        if self.fused:
            a = self.chain_a.forward(a)
            if self.pool5_split is not None:
                e.MaxPool2DSplit(a, None, self.pool5_split, (2, 2), (1, 0, 1, 0), (1, 1))
                return self.chain_b.forward(None, self.pool5_split)
            e.MaxPool2D(a, self.pool[5], (2, 2), (1, 0, 1, 0), (1, 1))
            return self.chain_b.forward(self.pool[5])
        for i in range(9):
            alpha = 1.0 if i == 8 else 0.1      # the last layer is LeakyRelu(1.0) in the reference graph
            e.Conv2d(a, self.w[i], self.conv[i], pad=(self.k[i] // 2, self.k[i] // 2), bias=self.b[i], act="leaky",
                     alpha=alpha)
            a = self.conv[i]
            if i < 5:
                e.MaxPool2D(a, self.pool[i], (2, 2), (0, 0), (2, 2))
                a = self.pool[i]
            elif i == 5:
                e.MaxPool2D(a, self.pool[i], (2, 2), (1, 0, 1, 0), (1, 1))
                a = self.pool[i]
        return self.out

    @property
    def flops_per_sample(self):
        s, f = self.size, 0
        for i in range(9):
            f += 2 * s * s * self.ch[i + 1] * self.ch[i] * self.k[i] ** 2
            if i < 5:
                s //= 2
        return f

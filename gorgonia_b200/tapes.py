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
`fused=True` uses the fused bias/activation stores of b200_gemm / b200_conv2d_fwd and, where a
2x2/2 pool follows a convolution, b200_conv2d_maxpool_fwd (the convolution output is then never
materialised); `fused=False` issues one engine call per reference instruction and leaves fusing to
the engine's deferred queue.
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

    def forward(self):
        e, a = self.e, self.x
        for i in range(3):
            last = i == 2
            if self.fused:
                e.MatMul(a, self.w[i], self.h[i], bias=self.b[i], bias_kind="col", act=None if last else "rectify")
            else:
                e.MatMul(a, self.w[i], self.h[i])
                e.BroadcastBinary("add", self.h[i], self.b[i], 1, self.DIMS[i + 1], unsafe=True)
                if not last:   # Rectify (nn.go:154-162): gte(x, 0) as float, then mul
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
        self.pool = [e.empty((batch, self.CH[i + 1], hw[i] // 2, hw[i] // 2)) for i in range(3)]
        self.fc = e.empty((batch, 625))
        self.fmask = None if fused else e.empty((batch, 625))
        self.logits = e.empty((batch, 10))
        self.out = e.empty((batch, 10))

    def forward(self):
        e, a = self.e, self.x
        for i in range(3):
            if self.fused:
                e.Conv2dMaxPool(a, self.wc[i], self.pool[i], pad=(1, 1), act="rectify")
            else:
                e.Conv2d(a, self.wc[i], self.conv[i], pad=(1, 1))
                e.GteScalar(self.conv[i], 0.0, reuse=self.cmask[i])
                e.Mul(self.conv[i], self.cmask[i], unsafe=True)
                e.MaxPool2D(self.conv[i], self.pool[i], (2, 2), (0, 0), (2, 2))
            a = self.pool[i]
        flat = a.reshape(self.batch, 1152)
        if self.fused:
            e.MatMul(flat, self.wd[0], self.fc, act="rectify")
        else:
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
            self.conv.append(None if fused and i < 5 else e.empty((batch, ch[i + 1], s, s)))
            if i < 5:
                s //= 2
                self.pool.append(e.empty((batch, ch[i + 1], s, s)))
            elif i == 5:
                self.pool.append(e.empty((batch, ch[i + 1], s, s)))
        self.out = self.conv[8]

    def forward(self):
        e, a = self.e, self.x
        for i in range(9):
            alpha = 1.0 if i == 8 else 0.1      # the last layer is LeakyRelu(1.0) in the reference graph
            if self.fused and i < 5:
                e.Conv2dMaxPool(a, self.w[i], self.pool[i], pad=(1, 1), bias=self.b[i], act="leaky", alpha=alpha)
                a = self.pool[i]
                continue
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

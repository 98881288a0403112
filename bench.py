#!/usr/bin/env python
"""Benchmark of the B200 engine on gorgonia's hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line (rank 0). Workloads (--workload):
  yolo         (default) forward pass of tiny-YOLOv2, batch 64 of 3x416x416 images sharded by batch
               over the ranks, weights replicated, no collective. Metric: samples/s.
  mlp | lenet  the other two inference graphs, batch 256 / 8192, sharded the same way.
  elementwise  the float32 elementwise / broadcast / fused-chain sweep on vectors of 2^29
               elements. One step = Add, Mul, Sub, Div, Pow, Gt (12 B/elem each), Exp, Tanh, Sigmoid
               (8 B/elem), broadcast Add of (B,1024)+(1,1024) (8 B/elem) and the fused chain
               tanh(x*w+b) (16 B/elem). Metric: GB/s of algorithmic bytes. N GPUs = N replicas.
               As the headline it also reports the sweep at 2^20, 2^24 and 2^27 elements, the
               broadcast Add for B = 4096 .. 262144 and the chain with (1,1024) rows for w and b.
  gemm         MatMul M=N=K=8192, float32 (3xTF32). Metric: TFLOP/s (2*M*N*K). Replicas.
  linalg       the whole GEMM/GEMV sweep: MatMul 1024^3, 4096^3, 8192^3 in float32 and bfloat16, a
               batch of 64 products of 512^3, MatVecMul 16384^2 in both orientations, Outer 8192^2,
               each with its own roofline. Headline value: the 8192^3 float32 product.
  backward     the backward ops and BatchNorm.
Unless --no-others is given, the line also carries short measurements of the other workloads
under "other_workloads" (so one run reports samples/s, GB/s and TFLOP/s).

Every workload checks what it timed: after the timed region, outside it, a sample of the result
is compared with the CPU oracle on the same inputs ("parity_checked" in the workload's object).
A run whose check fails raises instead of printing a throughput.

`value` is measured with the inputs resident in HBM; `e2e` is the same step driven through the
C ABI from pinned host buffers: host->device copies of the step's inputs and a device->host read
of the step's result inside the timed region.

With --impl reference the same step runs on the host cores through the CPU oracle (the
restatement of gorgonia's CPU engine; the Go reference itself cannot be built here), on a bounded
sample of the workload.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ELEMENTWISE_OPS = [  # (name, kind, algorithmic bytes per element)
    ("add", "bin", 12), ("mul", "bin", 12), ("sub", "bin", 12), ("div", "bin", 12), ("pow", "bin", 12),
    ("gt", "bin", 12), ("exp", "un", 8), ("tanh", "un", 8), ("sigmoid", "un", 8),
    ("bcast_add", "bcast", 8), ("chain_tanh_xw_b", "chain", 16),
]
BYTES_PER_ELEM_STEP = sum(b for _, _, b in ELEMENTWISE_OPS)
MODEL_BATCH = {"mlp": 256, "lenet": 8192, "yolo": 64}
REF_NOTE = ("CPU restatement of gorgonia's CPU-engine semantics (oracle/); the Go reference cannot be built here "
            "(no Go toolchain, dependencies not vendored)")


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def host_threads():
    """Cores this process may use. Launchers export OMP_NUM_THREADS=1 to their children, which would
    make the CPU legs single-threaded under torchrun: the oracle's thread count is set explicitly."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def oracle_all_cores():
    from oracle import oracle
    oracle.set_threads(host_threads())
    return oracle


class ParityError(AssertionError):
    pass


def _ratio_gemm(got, want, rel):
    """max |g - r| / (rel * max(|r|, rms(r))): <= 1 passes (the tolerance of the parity tests)."""
    g = np.asarray(got, dtype=np.float64)
    r = np.asarray(want, dtype=np.float64)
    rms = float(np.sqrt(np.mean(r * r))) if r.size else 0.0
    lim = rel * np.maximum(np.abs(r), max(rms, 1e-300))
    return float((np.abs(g - r) / lim).max()) if r.size else 0.0


def _ratio_pointwise(got, want, rel=1e-6):
    g = np.asarray(got, dtype=np.float64)
    r = np.asarray(want, dtype=np.float64)
    tiny = float(np.finfo(np.float32).tiny)
    with np.errstate(invalid="ignore"):
        ok_special = (np.isnan(g) & np.isnan(r)) | (np.isinf(r) & (g == r))
        q = np.abs(g - r) / (rel * np.maximum(np.abs(r), tiny))
    q = np.where(ok_special, 0.0, q)
    return float(np.nan_to_num(q, nan=np.inf).max()) if q.size else 0.0


def _ratio_bits(got, want):
    g = np.ascontiguousarray(got).view(np.uint32)
    r = np.ascontiguousarray(want).view(np.uint32)
    differ = (g != r) & ~(np.isnan(got) & np.isnan(want))
    return float("inf") if differ.any() else 0.0


def parity_result(what, ratio, **kw):
    if not (ratio <= 1.0):
        raise ParityError(f"parity check failed for {what}: error is {ratio:.3g} x the tolerance")
    return dict({"max_err_over_tol": round(ratio, 4)}, **kw)


def read_slice(e, t, lo, count, dtype=np.float32):
    """Elements [lo, lo + count) of a device tensor, through the synchronous copy of the C ABI."""
    from gorgonia_b200._lib import check, lib
    out = np.empty(count, dtype=dtype)
    check(lib.b200_memcpy_d2h(e.h, out.ctypes.data, t.ptr + lo * out.itemsize, out.nbytes), e.h)
    return out


def sampled_product_ratio(got_rows, got_cols, a, b, rows, cols, rel):
    """One row and one column per tile of a product computed on the device, against the oracle."""
    oracle = oracle_all_cores()
    wr = oracle.gemm(np.ascontiguousarray(a[rows]), b)
    wc = oracle.gemm(a, np.ascontiguousarray(b[:, cols]))
    rms = float(np.sqrt(np.mean(wr.astype(np.float64) ** 2)))
    worst = 0.0
    for g_, w_ in ((got_rows, wr), (got_cols, wc)):
        lim = rel * np.maximum(np.abs(w_.astype(np.float64)), rms)
        worst = max(worst, float((np.abs(g_.astype(np.float64) - w_) / lim).max()))
    return worst


_TF32_PEAK = {}


def tf32_peak(e, pk):
    """TF32 tensor peak measured on this GPU by the library's own issue-only kernel; the assumed
    figure (measured bf16 burst / 2) only if that measurement fails."""
    key = e.device
    if key not in _TF32_PEAK:
        try:
            v = e.tf32_peak(2048)
            _TF32_PEAK[key] = (v, "measured here: back-to-back tcgen05.mma kind::tf32 128x256x8 on all SMs, "
                                  "operands in shared memory, no loads, no epilogue (b200_tf32_peak)")
        except Exception as ex:  # noqa: BLE001
            _TF32_PEAK[key] = (pk["bf16_tflops"] / 2, f"assumed: {pk['source']} bf16 burst / 2 ({str(ex)[:80]})")
    return _TF32_PEAK[key]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            time.sleep(0.05)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
                pw.append(float(f[2]))
            except ValueError:
                continue
            for k, nm in enumerate(names):
                if f[3 + k].lower().startswith("active"):
                    reasons.add(nm)
        load = sorted(sm)[len(sm) // 2:] if sm else []   # the busiest half stands for "under load"
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


class Ctx:
    """One rank: its engine, the rendezvous with the other ranks, device timing."""

    def __init__(self, args):
        import torch
        self.torch = torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.dist = None
        if self.world > 1:
            # NCCL_DEBUG=VERSION makes NCCL print a banner on stdout, where the one JSON line belongs
            if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
                os.environ["NCCL_DEBUG"] = "WARN"
            import torch.distributed as dist
            torch.cuda.set_device(self.local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist
        self.engine = None
        self.pairs = not getattr(args, "no_pairs", False)

    def make_engine(self, arena_bytes):
        from gorgonia_b200 import Engine
        if self.engine is not None:
            self.engine.Close()
        self.engine = Engine(device=self.local_rank, arena_bytes=int(arena_bytes), pairs=self.pairs)
        self.ev = (self.engine.event(), self.engine.event())
        self._flush = None
        return self.engine

    FLUSH_BYTES = 256 << 20   # twice the 126 MB L2

    def flush_l2(self):
        """Overwrites a buffer larger than L2, so that the next step finds none of its operands cached."""
        from gorgonia_b200._lib import check, lib
        e = self.engine
        if self._flush is None:
            self._flush = e.empty(self.FLUSH_BYTES // 4)
        check(lib.b200_memset(e.h, self._flush.ptr, 0, self.FLUSH_BYTES), e.h)

    def timed_flushed(self, step, steps, warmup, solo=False):
        """For operands that fit in L2: every timed step is bracketed by its own pair of events and
        preceded by an L2 flush that is not timed. Returns seconds per step: the max over ranks, or
        with `solo` this rank's own (side measurements that only rank 0 makes)."""
        e = self.engine
        evs = [(e.event(), e.event()) for _ in range(steps)]
        for _ in range(warmup):
            step()
        e.Signal() if solo else self.barrier()
        for a, b in evs:
            self.flush_l2()
            e.record(a)
            step()
            e.record(b)
        e.Signal() if solo else self.barrier()
        ms = sum(e.elapsed_ms(a, b) for a, b in evs)
        from gorgonia_b200._lib import lib
        for a, b in evs:
            lib.b200_event_destroy(e.h, a)
            lib.b200_event_destroy(e.h, b)
        return (ms if solo else self.max_over_ranks(ms)) / 1e3 / steps

    def barrier(self):
        self.engine.Signal()
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        if self.dist is None:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, step, steps, warmup, sampler=None):
        """W untimed steps, then exactly K steps between barriers; CUDA events on the engine's
        stream; max over ranks. Returns (seconds per step, kernel launches in the timed region)."""
        e = self.engine
        for _ in range(warmup):
            step()
        self.barrier()
        if sampler is not None and self.rank == 0:
            sampler.start()
        l0 = e.launches
        e.record(self.ev[0])
        for _ in range(steps):
            step()
        e.record(self.ev[1])
        self.barrier()
        ms = self.max_over_ranks(e.elapsed_ms(*self.ev))
        return ms / 1e3 / steps, e.launches - l0

    def pinned(self, arr):
        e = self.engine
        p = e.host_alloc(arr.nbytes)
        ct = {4: C.c_float, 8: C.c_double}[arr.dtype.itemsize]
        v = np.ctypeslib.as_array(C.cast(p, C.POINTER(ct)), shape=arr.shape)
        v[...] = arr
        return p, v

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()
        if self.engine is not None:
            self.engine.Close()


# ------------------------------------------------------------------------------------------
# elementwise sweep
# ------------------------------------------------------------------------------------------

def make_inputs(n, seed=2024):
    """x, y ~ N(0,1); Pow base = |x| + 0.1; a row of 1024 for the broadcast form."""
    g = np.random.Generator(np.random.Philox(seed))
    x = g.standard_normal(n, dtype=np.float32)
    y = g.standard_normal(n, dtype=np.float32)
    row = g.standard_normal(1024, dtype=np.float32)
    return x, y, row


def gpu_sweep_ops(e, T):
    x, y, base, row, r = T["x"], T["y"], T["base"], T["row"], T["r"]
    return {
        "add": lambda: e.Add(x, y, reuse=r), "mul": lambda: e.Mul(x, y, reuse=r),
        "sub": lambda: e.Sub(x, y, reuse=r), "div": lambda: e.Div(x, y, reuse=r),
        "pow": lambda: e.Pow(base, y, reuse=r), "gt": lambda: e.Gt(x, y, reuse=r),
        "exp": lambda: e.Unary("exp", x, reuse=r), "tanh": lambda: e.Unary("tanh", x, reuse=r),
        "sigmoid": lambda: e.Unary("sigmoid", x, reuse=r),
        "bcast_add": lambda: e.BroadcastBinary("add", x, row, 1, 1024, reuse=r),
        # tanh(x*w+b) with full-size w, b: three engine calls, one kernel
        "chain_tanh_xw_b": lambda: (e.Mul(x, y, reuse=r), e.Add(r, base, unsafe=True),
                                    e.Unary("tanh", r, unsafe=True)),
    }


def gpu_sweep_step(e, ops):
    """One step: 11 engine-level operations, flushed one by one so that each is its own kernel
    (the chain's three calls fuse into one)."""
    for name, _, _ in ELEMENTWISE_OPS:
        ops[name]()
        e.DoWork()


def cpu_sweep_step(oracle, x, y, base, row):
    oracle.binary("add", x, y); oracle.binary("mul", x, y); oracle.binary("sub", x, y)
    oracle.binary("div", x, y); oracle.binary("pow", base, y); oracle.binary("gt", x, y)
    oracle.unary("exp", x); oracle.unary("tanh", x); oracle.unary("sigmoid", x)
    oracle.binary_bcast("add", x, row, 1, 1024)
    return oracle.unary("tanh", oracle.binary("add", oracle.binary("mul", x, y), base))


def cpu_elementwise(steps, warmup, n_sample=1 << 24):
    oracle = oracle_all_cores()
    x, y, row = make_inputs(n_sample)
    base = (np.abs(x) + np.float32(0.1)).astype(np.float32)
    for _ in range(warmup):
        cpu_sweep_step(oracle, x, y, base, row)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_sweep_step(oracle, x, y, base, row)
    dt = (time.perf_counter() - t0) / steps
    return {"value": BYTES_PER_ELEM_STEP * n_sample / dt / 1e9, "unit": "GB/s", "cores": oracle.threads(),
            "kind": "port", "sample": f"{steps} steps of the same 11-op sweep on vectors of 2^24 float32 elements",
            "ms_per_step": dt * 1e3}


def Tensor_view(e, t, count):
    """The first `count` elements of a device tensor as a tensor of their own (no copy)."""
    from gorgonia_b200.engine import Tensor
    return Tensor(e, t.ptr, (count,), t.dtype, owned=False)


EXACT_OPS = ("add", "mul", "sub", "div", "gt", "bcast_add")   # correctly rounded or 0/1: bit-exact


def parity_elementwise(e, ops, r, hview, row, n, window=1 << 16):
    """Runs every op of the sweep once more and compares three windows of its result (start, an odd
    offset in the middle, end) with the oracle on the same windows of the inputs."""
    oracle = oracle_all_cores()
    window = min(window, n)
    starts = sorted({0, max(0, (n // 2 + 3) // 1024 * 1024), max(0, (n - window) // 1024 * 1024)})
    worst, worst_op = 0.0, None
    for name, kind, _ in ELEMENTWISE_OPS:
        ops[name]()
        e.DoWork()
        for lo in starts:
            got = read_slice(e, r, lo, window)
            x, y, base = (np.array(hview[k][lo:lo + window]) for k in ("x", "y", "base"))
            if name == "pow":
                want = oracle.binary("pow", base, y)
            elif kind == "bin":
                want = oracle.binary(name, x, y)
            elif kind == "un":
                want = oracle.unary(name, x)
            elif kind == "bcast":
                want = oracle.binary_bcast("add", x, row, 1, 1024)   # window starts are multiples of 1024
            else:
                want = oracle.unary("tanh", oracle.binary("add", oracle.binary("mul", x, y), base))
            q = _ratio_bits(got, want) if name in EXACT_OPS else _ratio_pointwise(got, want, 1e-6)
            if q > worst:
                worst, worst_op = q, name
    return parity_result(f"elementwise op {worst_op}", worst, ops=len(ELEMENTWISE_OPS),
                         elements_per_op=window * len(starts),
                         tolerance="bit-exact for add/mul/sub/div/gt/broadcast add, 1e-6 relative otherwise")


def wl_elementwise(ctx, args, main):
    n = args.elements if main else min(args.elements, 1 << 27)
    steps, warmup = (args.steps, args.warmup) if main else (5, 3)
    e = ctx.make_engine((4.25 if (args.profile or not main) else 8.5) * 4 * n + (64 << 20) + ctx.FLUSH_BYTES)
    x, y, row = make_inputs(n, seed=2024 + ctx.rank)
    base = (np.abs(x) + np.float32(0.1)).astype(np.float32)
    T = {"x": e.empty(n), "y": e.empty(n), "base": e.empty(n), "r": e.empty(n), "row": e.tensor(row)}
    host, hview = {}, {}
    for k, a in (("x", x), ("y", y), ("base", base)):
        host[k], hview[k] = ctx.pinned(a)
        e.copy_h2d_async(T[k], host[k])
    hout = e.host_alloc(4 * n)
    del x, y, base
    ops = gpu_sweep_ops(e, T)
    sampler = ClockSampler(ctx.local_rank)
    step_s, launches = ctx.timed(lambda: gpu_sweep_step(e, ops), steps, warmup, sampler)
    clocks = sampler.stop() if ctx.rank == 0 else None
    bytes_step = BYTES_PER_ELEM_STEP * n
    res = {"metric": "elementwise sweep throughput (algorithmic bytes)", "unit": "GB/s",
           "value": ctx.world * bytes_step / step_s / 1e9, "ms_per_step": step_s * 1e3, "dtype": "f32",
           "config": {"workload": "elementwise_sweep_f32", "elements": n, "ops": [o for o, _, _ in ELEMENTWISE_OPS],
                      "bytes_per_element_step": BYTES_PER_ELEM_STEP, "l2": "inputs larger than L2",
                      "parallelism": f"replicas x{ctx.world}" if ctx.world > 1 else "single GPU"},
           "gpu_launches": launches, "clocks": clocks, "steps": steps, "warmup": warmup}
    pk = peaks()
    achieved = bytes_step / step_s / 1e9     # 11 launches back to back: bytes per launch / time per launch
    res["roofline"] = {"bound": "hbm", "kernel": "pw_stream_kernel", "achieved": achieved, "peak": pk["hbm_gbs"],
                       "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "peak_source": pk["source"],
                       "frac_of_nominal_8TBs": achieved / 8000.0,
                       # dram__bytes_read + dram__bytes_write per launch, averaged over the 11 launches
                       # of a step: 113.35 bytes per element and step measured by ncu at 2^26 elements
                       # (profiles/pw_stream_kernel_elementwise_sweep_2p26.txt), scaled by element count
                       "traffic": 113.35 * n / len(ELEMENTWISE_OPS),
                       "algorithmic_bytes_per_launch": bytes_step / len(ELEMENTWISE_OPS),
                       "traffic_source": "ncu at 2^26 elements, scaled by element count"}
    if args.profile:
        return res
    if ctx.rank == 0:
        res["parity_checked"] = parity_elementwise(e, ops, T["r"], hview, row, n)
    if not main:
        return res
    # per-op breakdown (outside the headline region; each op bracketed by its own events)
    per_op = {}
    if ctx.rank == 0:
        for name, _, bpe in ELEMENTWISE_OPS:
            ops[name](); e.DoWork()
            e.record(ctx.ev[0])
            for _ in range(5):
                ops[name](); e.DoWork()
            e.record(ctx.ev[1])
            per_op[name] = round(bpe * n / (e.elapsed_ms(*ctx.ev) / 5 / 1e3) / 1e9, 1)
        # the chain with w and b as (1,1024) rows: 8 bytes per element (the reference would move 32)
        row2 = e.tensor((row * np.float32(0.5)).astype(np.float32))

        def chain_rows():
            e.BroadcastBinary("mul", T["x"], T["row"], 1, 1024, reuse=T["r"])
            e.BroadcastBinary("add", T["r"], row2, 1, 1024, unsafe=True)
            e.Unary("tanh", T["r"], unsafe=True)
            e.DoWork()
        chain_rows()
        l0 = e.launches
        e.record(ctx.ev[0])
        for _ in range(5):
            chain_rows()
        e.record(ctx.ev[1])
        per_op["chain_tanh_xw_b_rows"] = round(8 * n / (e.elapsed_ms(*ctx.ev) / 5 / 1e3) / 1e9, 1)
        res["roofline"]["chain_rows_launches_per_step"] = (e.launches - l0) // 5
    res["roofline"]["per_op_gbs"] = per_op
    res["per_op_gbs"] = per_op
    # the sweep at the config's smaller sizes and the broadcast Add over its B range; operands that
    # fit in L2 are flushed out before every timed step
    if ctx.rank == 0:
        sizes = {}
        for lg in (20, 24, 27):
            m_ = 1 << lg
            Ts = {k: Tensor_view(e, T[k], m_) for k in ("x", "y", "base", "r")}
            Ts["row"] = T["row"]
            ops_s = gpu_sweep_ops(e, Ts)
            s_ = ctx.timed_flushed(lambda: gpu_sweep_step(e, ops_s), 5, 2, solo=True)
            sizes[f"2^{lg}"] = round(BYTES_PER_ELEM_STEP * m_ / s_ / 1e9, 1)
        res["roofline"]["sweep_gbs_by_elements"] = sizes
        bsweep = {}
        for B in (4096, 8192, 16384, 32768, 65536, 131072, 262144):
            m_ = B * 1024
            xs, rs = Tensor_view(e, T["x"], m_), Tensor_view(e, T["r"], m_)

            def bstep():
                e.BroadcastBinary("add", xs, T["row"], 1, 1024, reuse=rs)
                e.DoWork()
            s_ = ctx.timed_flushed(bstep, 5, 2, solo=True)
            bsweep[str(B)] = round(8 * m_ / s_ / 1e9, 1)
        res["roofline"]["bcast_add_gbs_by_rows"] = bsweep

    # End to end: every step uploads its three input vectors from pinned host memory and reads its
    # result back, copies inside the timed region. Two sets of device buffers are used in turn: the
    # upload of step i+1 (copy stream, host to device) runs while step i computes and sends its result
    # back (compute stream, device to host), so the two directions of the link are busy together.
    T2 = {"x": e.empty(n), "y": e.empty(n), "base": e.empty(n), "r": e.empty(n), "row": T["row"]}
    sets, ops2 = (T, T2), (ops, gpu_sweep_ops(e, T2))
    state = {"i": 0}
    e.Signal()
    for k in ("x", "y", "base"):
        e.upload_async(sets[0][k], host[k])

    def e2e_step():
        i = state["i"]
        cur = i % 2
        e.upload_wait()                                   # this step's inputs have arrived in sets[cur]
        for k in ("x", "y", "base"):
            e.upload_async(sets[1 - cur][k], host[k])     # the next step's inputs start moving now
        gpu_sweep_step(e, ops2[cur])
        e.copy_d2h_async(hout, sets[cur]["r"])
        state["i"] = i + 1

    e2e_steps = max(2, min(steps, 5))
    e2e_s, _ = ctx.timed(e2e_step, e2e_steps, 2)
    res["e2e"] = {"value": ctx.world * bytes_step / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 3 * 4 * n,
                  "d2h_bytes_per_step": 4 * n, "steps": e2e_steps,
                  "note": "upload of the next step's inputs overlaps this step's kernels and its read-back"}
    return res


# ------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------

def parity_product(e, tc, a, b, rel, batch_index=None):
    """tc = a @ b on the device (row-major M x N, or entry `batch_index` of a batch). Reads back one
    row and one column per 128-wide tile and compares them with the oracle."""
    from gorgonia_b200._lib import check, lib
    M, N = a.shape[0], b.shape[1]
    g = np.random.Generator(np.random.Philox(4242))
    rows = np.array([min(M - 1, t * 128 + int(g.integers(128))) for t in range((M + 127) // 128)])
    cols = np.array([min(N - 1, t * 128 + int(g.integers(128))) for t in range((N + 127) // 128)])
    base = 0 if batch_index is None else batch_index * M * N
    got_rows = np.stack([read_slice(e, tc, base + int(r) * N, N) for r in rows])
    strip = read_columns(e, tc, base, cols, M, N)
    q = sampled_product_ratio(got_rows, strip, a, b, rows, cols, rel)
    return parity_result("matrix product", q, rows=len(rows), columns=len(cols),
                         tolerance=f"{rel:g} * max(|r|, rms(r))")


def read_columns(e, t, base, cols, M, N):
    """Columns `cols` of a row-major M x N device matrix, gathered on the device (ByIndices along
    axis 1 of the matrix viewed as (M, N, 1)) and read back as an M x len(cols) array."""
    from gorgonia_b200.engine import Tensor
    idx = e.tensor(np.asarray(cols, np.int64))
    out = e.empty((M, len(cols)))
    view = Tensor(e, t.ptr + base * 4, (M, N, 1), np.float32, owned=False)
    e.ByIndices(view, idx, out, axis=1)
    strip = out.numpy()
    idx.free()
    out.free()
    return strip


def wl_gemm(ctx, args, main):
    n = 8192
    steps, warmup = (args.steps, args.warmup) if main else (5, 3)
    e = ctx.make_engine(16 * 4 * n * n + (768 << 20))
    g = np.random.Generator(np.random.Philox(3 + ctx.rank))
    a = (g.standard_normal((n, n), dtype=np.float32) * np.float32(0.02))
    b = (g.standard_normal((n, n), dtype=np.float32) * np.float32(0.02))
    ta, tb, tc = e.empty((n, n)), e.empty((n, n)), e.empty((n, n))
    ha, _ = ctx.pinned(a)
    hb, _ = ctx.pinned(b)
    hc = e.host_alloc(4 * n * n)
    e.copy_h2d_async(ta, ha)
    e.copy_h2d_async(tb, hb)
    sampler = ClockSampler(ctx.local_rank)
    step_s, launches = ctx.timed(lambda: e.MatMul(ta, tb, tc), steps, warmup, sampler)
    clocks = sampler.stop() if ctx.rank == 0 else None
    flops = 2.0 * n ** 3
    pk = peaks()
    tf = flops / step_s / 1e12
    peak32, peak32_src = tf32_peak(e, pk)
    parity = None
    if ctx.rank == 0 and not args.profile:
        parity = parity_product(e, tc, a, b, 1e-5)
    res = {"metric": "MatMul float32 (3xTF32) throughput, 2*M*N*K", "unit": "TFLOP/s", "value": ctx.world * tf,
           "ms_per_step": step_s * 1e3, "dtype": "f32 (3xTF32 on tensor cores, fp32 accumulate)",
           "config": {"workload": "gemm_f32_8192", "M": n, "N": n, "K": n, "l2": "operands larger than L2",
                      "parallelism": f"replicas x{ctx.world}" if ctx.world > 1 else "single GPU"},
           "gpu_launches": launches, "clocks": clocks, "steps": steps, "warmup": warmup,
           "parity_checked": parity,
           "roofline": {"bound": "tensor", "kernel": "gemm_tc_kernel<3,128>", "achieved": 3 * tf,
                        "peak": peak32, "unit": "TFLOP/s (TF32 issued = 3 x algorithmic)",
                        "frac": 3 * tf / peak32, "peak_source": peak32_src,
                        "frac_of_bf16_burst_over_2": 3 * tf / (pk["bf16_tflops"] / 2), "traffic": None}}
    if not main or args.profile:
        # bf16 beside it, same shape
        tab, tbb = e.tensor_bf16(a), e.tensor_bf16(b)
        s2, _ = ctx.timed(lambda: e.MatMul(tab, tbb, tc), steps, warmup)
        res["bf16_tflops"] = ctx.world * flops / s2 / 1e12
        res["bf16_frac_of_measured_peak"] = flops / s2 / 1e12 / pk["bf16_tflops"]
        return res

    # two operand sets in turn: the upload of step i+1 overlaps the product and the read-back of step i
    ta2, tb2 = e.empty((n, n)), e.empty((n, n))
    sets = ((ta, tb), (ta2, tb2))
    state = {"i": 0}
    e.Signal()
    e.upload_async(ta, ha)
    e.upload_async(tb, hb)

    def e2e_step():
        i = state["i"]
        a_, b_ = sets[i % 2]
        e.upload_wait()
        e.upload_async(sets[(i + 1) % 2][0], ha)
        e.upload_async(sets[(i + 1) % 2][1], hb)
        e.MatMul(a_, b_, tc)
        e.copy_d2h_async(hc, tc)
        state["i"] = i + 1

    e2e_s, _ = ctx.timed(e2e_step, max(2, min(steps, 5)), 2)
    res["e2e"] = {"value": ctx.world * flops / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": 8 * n * n,
                  "d2h_bytes_per_step": 4 * n * n,
                  "note": "upload of the next step's operands overlaps this step's product and its read-back"}
    return res


def wl_linalg(ctx, args, main):
    """The GEMM/GEMV sweep of the configs: the 8192^3 float32 product is the headline (timed exactly
    like --workload gemm, with its end-to-end leg); every other item is timed with an L2 flush before
    each step and carries its own roofline and parity check."""
    res = wl_gemm(ctx, args, main)
    if args.profile:
        return res
    e = ctx.engine
    e.Signal()
    e.ResetAllocator()
    ctx._flush = None
    pk = peaks()
    peak32, peak32_src = tf32_peak(e, pk)
    steps = 5
    items = {"matmul_f32_8192": {"tflops": round(res["value"] / ctx.world, 1), "frac": round(res["roofline"]["frac"], 4),
                                 "bound": "tensor (3 x TF32 issued)", "parity_checked": res.get("parity_checked")}}
    g = np.random.Generator(np.random.Philox(31 + ctx.rank))

    def normal(shape):
        return g.standard_normal(shape, dtype=np.float32) * np.float32(0.02)

    from gorgonia_b200.engine import from_bf16, to_bf16
    for n in (1024, 4096, 8192):
        a, b = normal((n, n)), normal((n, n))
        tc = e.empty((n, n))
        flops = 2.0 * n ** 3
        if n != 8192:
            ta, tb = e.tensor(a), e.tensor(b)
            s_ = ctx.timed_flushed(lambda: e.MatMul(ta, tb, tc), steps, 3)
            tf = flops / s_ / 1e12
            items[f"matmul_f32_{n}"] = {"tflops": round(tf, 1), "frac": round(3 * tf / peak32, 4),
                                        "bound": "tensor (3 x TF32 issued)",
                                        "parity_checked": parity_product(e, tc, a, b, 1e-5) if ctx.rank == 0 else None}
            ta.free(); tb.free()
        ab, bb = from_bf16(to_bf16(a)), from_bf16(to_bf16(b))
        tab, tbb = e.tensor_bf16(ab), e.tensor_bf16(bb)
        s_ = ctx.timed_flushed(lambda: e.MatMul(tab, tbb, tc), steps, 3)
        tf = flops / s_ / 1e12
        items[f"matmul_bf16_{n}"] = {"tflops": round(tf, 1), "frac": round(tf / pk["bf16_tflops"], 4),
                                     "bound": "tensor (bf16, measured cuBLAS burst)",
                                     "parity_checked": parity_product(e, tc, ab, bb, 1e-2) if ctx.rank == 0 else None}
        e.Signal()
        e.ResetAllocator()
        ctx._flush = None
    # a batch of 64 independent 512^3 products in one launch
    A, Bm = normal((64, 512, 512)), normal((64, 512, 512))
    tA, tB, tC = e.tensor(A), e.tensor(Bm), e.empty((64, 512, 512))
    s_ = ctx.timed_flushed(lambda: e.MatMul(tA, tB, tC), steps, 3)
    tf = 64 * 2.0 * 512 ** 3 / s_ / 1e12
    items["matmul_f32_64x512"] = {"tflops": round(tf, 1), "frac": round(3 * tf / peak32, 4),
                                  "bound": "tensor (3 x TF32 issued)",
                                  "parity_checked": parity_product(e, tC, A[37], Bm[37], 1e-5, batch_index=37)
                                  if ctx.rank == 0 else None}
    e.Signal()
    e.ResetAllocator()
    ctx._flush = None
    # MatVecMul 16384 x 16384, both orientations: the matrix is read once
    n = 16384
    a, x = normal((n, n)), g.standard_normal(n, dtype=np.float32)
    ta, tx, ty = e.tensor(a), e.tensor(x), e.empty(n)
    oracle = oracle_all_cores() if ctx.rank == 0 else None
    for trans in (False, True):
        s_ = ctx.timed_flushed(lambda: e.MatVecMul(ta, tx, ty, transA=trans), steps, 3)
        gbs = 4.0 * (n * n + 2 * n) / s_ / 1e9
        par = None
        if ctx.rank == 0:
            par = parity_result("MatVecMul", _ratio_gemm(ty.numpy(), oracle.gemv(a, x, transA=trans), 1e-5),
                                elements=n, tolerance="1e-5 * max(|r|, rms(r))")
        items["matvecmul_16384" + ("_transposed" if trans else "")] = {
            "gbs": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 4), "bound": "hbm", "parity_checked": par}
    e.Signal()
    e.ResetAllocator()
    ctx._flush = None
    # Outer of two 8192-vectors: 268 MB written
    n = 8192
    x, y = g.standard_normal(n, dtype=np.float32), g.standard_normal(n, dtype=np.float32)
    tx, ty, to = e.tensor(x), e.tensor(y), e.empty((n, n))
    s_ = ctx.timed_flushed(lambda: e.Outer(tx, ty, to), steps, 3)
    gbs = 4.0 * n * n / s_ / 1e9
    par = None
    if ctx.rank == 0:
        rows = np.arange(0, n, 131)
        got = np.stack([read_slice(e, to, int(r) * n, n) for r in rows])
        par = parity_result("Outer", _ratio_bits(got, oracle.outer(x[rows], y)), rows=len(rows), tolerance="bit-exact")
    items["outer_8192"] = {"gbs": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 4), "bound": "hbm (write)",
                           "parity_checked": par}
    res["config"]["workload"] = "linalg_sweep (headline: gemm_f32_8192)"
    res["config"]["l2"] = "8192^3 operands larger than L2; every other item flushes L2 before each timed step"
    res["roofline"]["items"] = items
    res["roofline"]["tf32_peak"] = peak32
    res["roofline"]["tf32_peak_source"] = peak32_src
    return res


# ------------------------------------------------------------------------------------------
# backward ops (max-pool gradient, col2im, softmax derivative, Incr-mode MatMul)
# ------------------------------------------------------------------------------------------

BACKWARD_SHAPES = {"pool": (2048, 32, 28, 28), "col2im": (1024, 32, 14, 14), "softmax": (1 << 22, 10),
                   "batchnorm": (2048, 64, 14, 14)}


def wl_backward(ctx, args, main):
    """HBM-bound backward ops at LeNet's shapes; algorithmic bytes = every operand once."""
    steps, warmup = (args.steps, args.warmup) if main else (5, 3)
    e = ctx.make_engine(6 << 30)
    g = np.random.Generator(np.random.Philox(17 + ctx.rank))
    per_op, total_bytes, total_s, launches = {}, 0.0, 0.0, 0
    sampler = ClockSampler(ctx.local_rank)
    # max-pool gradient: dy + mask read, dx written
    B, Cc, H, W = BACKWARD_SHAPES["pool"]
    x = e.tensor(g.standard_normal((B, Cc, H, W), dtype=np.float32))
    y, mask = e.empty((B, Cc, H // 2, W // 2)), e.empty((B, Cc, H // 2, W // 2), np.int64)
    e.MaxPool2D(x, y, (2, 2), (0, 0), (2, 2), mask=mask)
    dx = x   # reuse the buffer
    s_, l_ = ctx.timed(lambda: e.MaxPool2DDiff(y, mask, dx, (2, 2), (0, 0), (2, 2)), steps, warmup, sampler)
    by = B * Cc * (H // 2) * (W // 2) * 12 + B * Cc * H * W * 4
    per_op["maxpool_bwd"] = by / s_ / 1e9
    total_bytes += by; total_s += s_; launches += l_
    e.ResetAllocator()
    # col2im: col read, image written
    B, Cc, H, W = BACKWARD_SHAPES["col2im"]
    col = e.tensor(g.standard_normal((B, H, W, Cc * 9), dtype=np.float32))
    im = e.empty((B, Cc, H, W))
    s_, l_ = ctx.timed(lambda: e.Col2Im(col, im, (3, 3), (1, 1)), steps, warmup)
    by = B * H * W * Cc * 9 * 4 + B * Cc * H * W * 4
    per_op["col2im"] = by / s_ / 1e9
    total_bytes += by; total_s += s_; launches += l_
    e.ResetAllocator()
    # softmax derivative: y + grad read, dx written
    R, L = BACKWARD_SHAPES["softmax"]
    ys = e.tensor(g.random((R, L), dtype=np.float32))
    gr = e.tensor(g.standard_normal((R, L), dtype=np.float32))
    dxs = e.empty((R, L))
    s_, l_ = ctx.timed(lambda: e.SoftMaxDiff(ys, gr, dxs), steps, warmup)
    by = R * L * 12
    per_op["softmax_bwd"] = by / s_ / 1e9
    total_bytes += by; total_s += s_; launches += l_
    e.ResetAllocator()
    # BatchNorm, training mode: x is read twice (the statistics must exist before the first output), y written
    B, Cc, H, W = BACKWARD_SHAPES["batchnorm"]
    xb = e.tensor(g.standard_normal((B, Cc, H, W), dtype=np.float32))
    yb = e.empty((B, Cc, H, W))
    rm, rv = e.tensor(np.zeros(Cc, np.float32)), e.tensor(np.ones(Cc, np.float32))
    sm, sv = e.empty((Cc,)), e.empty((Cc,))
    s_, l_ = ctx.timed(lambda: e.BatchNorm(xb, yb, rm, rv, sm, sv), steps, warmup)
    by = B * Cc * H * W * 12
    per_op["batchnorm_train"] = by / s_ / 1e9
    total_bytes += by; total_s += s_; launches += l_
    e.ResetAllocator()
    # Incr-mode MatMul, 4096^3
    n = 4096
    a = e.tensor((g.standard_normal((n, n), dtype=np.float32) * np.float32(0.02)))
    b = e.tensor((g.standard_normal((n, n), dtype=np.float32) * np.float32(0.02)))
    c = e.tensor(np.zeros((n, n), np.float32))
    s_, l_ = ctx.timed(lambda: e.MatMul(a, b, c, incr=True), steps, warmup)
    launches += l_
    clocks = sampler.stop() if ctx.rank == 0 else None
    pk = peaks()
    gbs = total_bytes / total_s / 1e9
    return {"metric": "backward ops throughput (algorithmic bytes)", "unit": "GB/s", "value": ctx.world * gbs,
            "ms_per_step": total_s * 1e3, "dtype": "f32",
            "config": {"workload": "backward_ops", "shapes": {k: list(v) for k, v in BACKWARD_SHAPES.items()},
                       "l2": "operands larger than L2",
                       "parallelism": f"replicas x{ctx.world}" if ctx.world > 1 else "single GPU"},
            "gpu_launches": launches, "clocks": clocks, "steps": steps, "warmup": warmup,
            "per_op_gbs": {k: round(v, 1) for k, v in per_op.items()},
            "matmul_incr_4096_tflops": 2.0 * n ** 3 / s_ / 1e12,
            "roofline": {"bound": "hbm", "kernel": "maxpool2x2_bwd_kernel + col2im_rows4_kernel + softmax_bwd_short_kernel + bn_*_kernel",
                         "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                         "peak_source": pk["source"], "traffic": None}}


# ------------------------------------------------------------------------------------------
# inference graphs
# ------------------------------------------------------------------------------------------

def model_input(name, batch, seed):
    g = np.random.Generator(np.random.Philox(seed))
    shape = {"mlp": (batch, 784), "lenet": (batch, 1, 28, 28), "yolo": (batch, 3, 416, 416)}[name]
    return g.random(shape, dtype=np.float32)


def make_model(name, e, batch):
    from gorgonia_b200 import tapes
    return {"mlp": tapes.MLP, "lenet": tapes.LeNet, "yolo": tapes.TinyYolo}[name](e, batch)


def dominant_kernel(ctx, name, m, b):
    """Times the launch that takes the largest share of a graph's step on its own: tiny-YOLO's layer 7
    (1024 -> 1024 channels on 13 x 13, conv_tma_kernel), LeNet's conv1 + pool (conv_win_kernel). Ten
    launches between CUDA events on the engine's stream, after the step itself has run."""
    if name == "mlp":
        return None
    e = ctx.engine
    if name == "yolo":
        chain, i, kern = m.chain_b, 1, "conv_tma_kernel<128, 32> (layer 7: 1024 -> 1024 channels, 3x3, 13x13)"
    else:
        chain, i, kern = m.chain, 1, "conv_win_kernel<64, 32> (conv1 + pool: 32 -> 64 channels, 3x3, 14x14)"
    L, prev = chain.layers[i], chain.layers[i - 1]
    x_split = prev["pool_split"] if prev.get("pool_split") is not None else prev["split"]
    x_plain = prev["pooled"] if prev.get("pooled") is not None else prev["y"]

    def launch():
        e.Conv2dChain(x_plain if x_split is None else None, L["w"], L["y"], L["in_shape"], pad=L["pad"], bias=L["bias"],
                      act=L["act"], alpha=L["alpha"], pool2=L["fuse_pool"], x_split=x_split, y_split=L["split"])
    launch()
    e.Signal()
    e.record(ctx.ev[0])
    for _ in range(10):
        launch()
    e.record(ctx.ev[1])
    us = e.elapsed_ms(*ctx.ev) * 100.0
    B, Cc, H, W = L["in_shape"]
    K, _, kh, kw = L["w"].shape
    flops = 2.0 * B * H * W * K * Cc * kh * kw        # stride 1, same padding
    out = {"kernel": kern, "us": us, "flops": flops, "tflops": flops / (us * 1e-6) / 1e12}
    if name == "yolo" and b == 64:
        out["traffic"] = 754.3e6
        out["traffic_source"] = ("dram__bytes_read.sum + dram__bytes_write.sum of this launch under ncu "
                                 "(profiles/conv_tma_kernel_yolo_layer7.txt)")
    return out


def parity_model(name, m, x):
    """Compares the device output of the batch just timed with the oracle running the same graph op
    by op on a sample of it: every sample of the MLP batch, 64 LeNet images spread over the batch,
    the first and the last tiny-YOLO image."""
    from oracle import graphs
    oracle_all_cores()
    b = x.shape[0]
    if name == "mlp":
        idx = np.arange(b)
    elif name == "lenet":
        k = min(64, b)
        g = np.random.Generator(np.random.Philox(99))
        idx = np.sort((np.arange(k) * (b // k) + g.integers(0, max(1, b // k), k)).astype(np.int64))
    else:
        idx = np.array(sorted({0, b - 1}))
    got = m.out.numpy()[idx]
    want = {"mlp": graphs.mlp, "lenet": graphs.lenet, "yolo": graphs.tiny_yolo}[name](m, np.ascontiguousarray(x[idx]))
    q = _ratio_gemm(got, want, 1e-5)
    if name != "yolo" and not np.array_equal(got.argmax(1), want.argmax(1)):
        q = float("inf")
    return parity_result(f"{name} forward", q, samples=int(len(idx)),
                         tolerance="1e-5 * max(|r|, rms(r)); argmax bit-exact")


def wl_model(ctx, args, name, main):
    from gorgonia_b200 import shard
    total = args.batch if (args.batch and main) else MODEL_BATCH[name]
    lo, hi = shard.my_shard(total, ctx.rank, ctx.world)
    b = hi - lo                                  # this rank's shard: strong scaling of a fixed batch
    steps, warmup = (args.steps, args.warmup) if main else (5, 3)
    arena = {"mlp": 1 << 30, "lenet": 8 << 30, "yolo": 24 << 30}[name]
    e = ctx.make_engine(arena)
    m = make_model(name, e, b)
    x = model_input(name, b, 77 + ctx.rank)
    hx, _ = ctx.pinned(x)
    hy = e.host_alloc(m.out.nbytes)
    e.copy_h2d_async(m.x, hx)
    # device-resident: one recorded tape per step
    m.record()
    sampler = ClockSampler(ctx.local_rank)
    step_s, launches = ctx.timed(m.replay, steps, warmup, sampler)
    clocks = sampler.stop() if ctx.rank == 0 else None
    pk = peaks()
    tf = m.flops_per_sample * b / step_s / 1e12
    peak32, peak32_src = tf32_peak(e, pk)
    parity = None
    if ctx.rank == 0 and not args.profile:
        parity = parity_model(name, m, x)
    dom = dominant_kernel(ctx, name, m, b) if not args.profile else None
    res = {"metric": f"{name} forward throughput", "unit": "samples/s", "value": total / step_s,
           "ms_per_step": step_s * 1e3, "dtype": "f32 (matrix products as 3xTF32, fp32 accumulate)",
           "config": {"workload": f"{name}_forward", "global_batch": total, "batch_per_gpu": b,
                      "parallelism": f"batch-sharded x{ctx.world}, weights replicated, no collective",
                      "l2": "activations larger than L2" if name != "mlp" else "flush not needed: launch-bound"},
           "gpu_launches": launches, "clocks": clocks, "steps": steps, "warmup": warmup, "scaling": "strong",
           "parity_checked": parity, "latency_us_per_batch": step_s * 1e6,
           "roofline": {"bound": "tensor",
                        "kernel": {"mlp": "gemm_tc_kernel (whole step)",
                                   "lenet": "conv_win_kernel + conv_tma_kernel + gemm_tc_kernel (whole step)",
                                   "yolo": "conv_tma_kernel + conv_win_kernel (whole step)"}[name],
                        "achieved": 3 * tf,
                        "peak": peak32, "unit": "TFLOP/s (TF32 issued = 3 x algorithmic)",
                        "frac": 3 * tf / peak32, "peak_source": peak32_src,
                        "frac_of_bf16_burst_over_2": 3 * tf / (pk["bf16_tflops"] / 2), "traffic": None}}
    if dom is not None:
        # the dominant kernel of the step, timed alone: its own launches between CUDA events
        whole = {k: res["roofline"][k] for k in ("kernel", "achieved", "frac")}
        res["roofline"].update({"kernel": dom["kernel"], "achieved": 3 * dom["tflops"], "frac": 3 * dom["tflops"] / peak32,
                                "us_per_launch": dom["us"], "share_of_step": dom["us"] * 1e-6 / step_s,
                                "algorithmic_flops_per_launch": dom["flops"], "traffic": dom.get("traffic"),
                                "traffic_source": dom.get("traffic_source"), "whole_step": whole})
    if args.profile:
        m.close()
        return res

    # End to end: every step uploads its input batch from pinned host memory and reads its result
    # back to the host. Two device staging buffers are used in turn, so the upload of batch i+1
    # (copy stream) hides behind the forward pass of batch i; each step is one recorded tape:
    # staging -> input, forward, result -> host.
    m.close()
    e.Signal()
    stage = [e.empty(m.x.shape), e.empty(m.x.shape)]
    from gorgonia_b200._lib import lib, check
    tapes_ab = []
    for sbuf in stage:
        e.tape_begin()
        check(lib.b200_memcpy_d2d(e.h, m.x.ptr, sbuf.ptr, m.x.nbytes), e.h)
        m.forward()
        e.copy_d2h_async(hy, m.out)
        tapes_ab.append(e.tape_end())
    state = {"i": 0}
    e.upload_async(stage[0], hx)

    def e2e_step():
        i = state["i"]
        e.upload_wait()                              # batch i has arrived in stage[i % 2]
        e.upload_async(stage[(i + 1) % 2], hx)       # batch i+1 starts uploading now
        e.tape_launch(tapes_ab[i % 2])
        state["i"] = i + 1

    e2e_s, _ = ctx.timed(e2e_step, max(2, min(steps, 10)), 2)
    for t in tapes_ab:
        e.tape_destroy(t)
    res["e2e"] = {"value": total / e2e_s, "unit": "samples/s", "h2d_bytes_per_step": int(x.nbytes),
                  "d2h_bytes_per_step": int(m.out.nbytes),
                  "note": "upload of the next batch overlaps the forward pass of the current one"}
    return res


def cpu_model(name, steps=1):
    from gorgonia_b200 import tapes  # host-side weight draws only; no engine is created
    from oracle import graphs
    oracle = oracle_all_cores()
    sample = {"mlp": 256, "lenet": 256, "yolo": 8}[name]

    class Host:  # a tape object without a device: just the seeded host weights
        pass

    g = np.random.Generator(np.random.Philox({"mlp": 286, "lenet": 5, "yolo": 9}[name]))
    h = Host()
    if name == "mlp":
        h.w_host = [tapes.glorot_uniform(g, (tapes.MLP.DIMS[i], tapes.MLP.DIMS[i + 1])) for i in range(3)]
        h.b_host = [np.zeros(tapes.MLP.DIMS[i + 1], np.float32) for i in range(3)]
        fn = graphs.mlp
    elif name == "lenet":
        ch = tapes.LeNet.CH
        h.wc_host = [tapes.he_normal(g, (ch[i + 1], ch[i], 3, 3), ch[i] * 9) for i in range(3)]
        h.wd_host = [tapes.he_normal(g, (1152, 625), 1152), tapes.he_normal(g, (625, 10), 625)]
        fn = graphs.lenet
    else:
        ch = tapes.TinyYolo.CH
        h.k = [3] * 8 + [1]
        h.w_host = [tapes.he_normal(g, (ch[i + 1], ch[i], h.k[i], h.k[i]), ch[i] * h.k[i] ** 2) for i in range(9)]
        h.b_host = [(g.standard_normal(ch[i + 1]) * 0.1).astype(np.float32) for i in range(9)]
        fn = graphs.tiny_yolo
    x = model_input(name, sample, 77)
    fn(h, x[:max(1, sample // 8)])           # warm-up on a slice
    t0 = time.perf_counter()
    for _ in range(steps):
        fn(h, x)
    dt = (time.perf_counter() - t0) / steps
    return {"value": sample / dt, "unit": "samples/s", "cores": oracle.threads(), "kind": "port",
            "sample": f"{steps} forward pass(es) of {sample} samples of the same graph", "ms_per_step": dt * 1e3}


def cpu_gemm(steps=1, n=1024):
    oracle = oracle_all_cores()
    g = np.random.Generator(np.random.Philox(3))
    a = (g.standard_normal((n, n), dtype=np.float32) * np.float32(0.02))
    b = (g.standard_normal((n, n), dtype=np.float32) * np.float32(0.02))
    oracle.gemm(a[:128], b)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.gemm(a, b)
    dt = (time.perf_counter() - t0) / steps
    return {"value": 2.0 * n ** 3 / dt / 1e12, "unit": "TFLOP/s", "cores": oracle.threads(), "kind": "port",
            "sample": f"{steps} MatMul(s) of {n}^3 float32 (double accumulation)", "ms_per_step": dt * 1e3}


def cpu_backward(steps=1):
    """The oracle's maxpool gradient, col2im, softmax derivative and batch-norm on 1/16 of the GPU leg's batches."""
    oracle = oracle_all_cores()
    g = np.random.Generator(np.random.Philox(17))
    B, Cc, H, W = BACKWARD_SHAPES["pool"]
    B //= 16
    x = g.standard_normal((B, Cc, H, W), dtype=np.float32)
    y, mask = oracle.maxpool2d(x, (2, 2), (0, 0), (2, 2))
    B2, C2, H2, W2 = BACKWARD_SHAPES["col2im"]
    B2 //= 16
    col = g.standard_normal((B2, H2, W2, C2 * 9), dtype=np.float32)
    R, L = BACKWARD_SHAPES["softmax"]
    R //= 16
    ys, gr = g.random((R, L), dtype=np.float32), g.standard_normal((R, L), dtype=np.float32)
    B3, C3, H3, W3 = BACKWARD_SHAPES["batchnorm"]
    B3 //= 16
    xb = g.standard_normal((B3, C3, H3, W3), dtype=np.float32)
    by = (B * Cc * (H // 2) * (W // 2) * 12 + B * Cc * H * W * 4 + B2 * H2 * W2 * C2 * 9 * 4 + B2 * C2 * H2 * W2 * 4 +
          R * L * 12 + B3 * C3 * H3 * W3 * 12)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.maxpool2d_bwd(y, mask, x.shape)
        oracle.col2im(col, (B2, C2, H2, W2), 3, 3, (1, 1))
        oracle.softmax_bwd(ys, gr)
        oracle.batchnorm(xb, np.zeros(C3, np.float32), np.ones(C3, np.float32))
    dt = (time.perf_counter() - t0) / steps
    return {"value": by / dt / 1e9, "unit": "GB/s", "cores": oracle.threads(), "kind": "port",
            "sample": f"{steps} pass(es) over 1/16 of the GPU leg's batches", "ms_per_step": dt * 1e3}


def cpu_leg(workload, steps, warmup):
    if workload == "backward":
        return cpu_backward(steps)
    if workload == "elementwise":
        return cpu_elementwise(steps, warmup)
    if workload in ("gemm", "linalg"):
        return cpu_gemm(steps)
    return cpu_model(workload, steps)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 3))
    c = cpu_leg(args.workload, steps, 1 if args.workload == "elementwise" else 0)
    line = {"impl": "reference", "metric": c.pop("metric", None), "value": c["value"], "unit": c["unit"],
            "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": c.pop("ms_per_step"),
            "higher_is_better": True, "scaling": "weak" if args.workload in ("elementwise", "gemm", "linalg", "backward") else "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": ({"workload": f"{args.workload}_forward", "global_batch": MODEL_BATCH[args.workload],
                        "sample": c["sample"]} if args.workload in MODEL_BATCH
                       else {"workload": args.workload, "sample": c["sample"]}),
            "cpu_baseline": c, "e2e": {"value": c["value"], "unit": c["unit"], "h2d_bytes_per_step": 0,
                                       "d2h_bytes_per_step": 0}, "note": REF_NOTE}
    line["metric"] = {"elementwise": "elementwise sweep throughput (algorithmic bytes)",
                      "backward": "backward ops throughput (algorithmic bytes)",
                      "gemm": "MatMul float32 (3xTF32) throughput, 2*M*N*K",
                      "linalg": "MatMul float32 (3xTF32) throughput, 2*M*N*K"}.get(args.workload,
                                                                         f"{args.workload} forward throughput")
    print(json.dumps(line), flush=True)


def run_workload(ctx, args, name, main):
    if name == "elementwise":
        return wl_elementwise(ctx, args, main)
    if name == "gemm":
        return wl_gemm(ctx, args, main)
    if name == "linalg":
        return wl_linalg(ctx, args, main)
    if name == "backward":
        return wl_backward(ctx, args, main)
    return wl_model(ctx, args, name, main)


def run_ours(args):
    ctx = Ctx(args)
    res = run_workload(ctx, args, args.workload, True)
    others = {}
    if not args.no_others and not args.profile:
        for name in ("yolo", "lenet", "mlp", "elementwise", "gemm", "backward"):
            if name == args.workload or (name == "gemm" and args.workload == "linalg"):
                continue
            try:
                r = run_workload(ctx, args, name, False)
                keep = {k: r[k] for k in ("metric", "value", "unit", "ms_per_step", "config", "roofline",
                                          "parity_checked", "latency_us_per_batch", "clocks") if k in r}
                for k in ("bf16_tflops", "bf16_frac_of_measured_peak", "per_op_gbs", "matmul_incr_4096_tflops"):
                    if k in r:
                        keep[k] = r[k]
                others[name] = keep
            except Exception as ex:  # a side measurement must not cost the headline
                others[name] = {"error": str(ex)[:200]}
    if ctx.rank == 0:
        line = {"metric": res["metric"], "value": res["value"], "unit": res["unit"], "n_gpus": ctx.world,
                "steps": res["steps"], "warmup": res["warmup"], "ms_per_step": res["ms_per_step"],
                "higher_is_better": True, "scaling": res.get("scaling", "weak"), "vs_baseline": None,
                "dtype": res["dtype"], "data": "synthetic", "config": res["config"], "roofline": res["roofline"],
                "e2e": res.get("e2e"), "gpu_launches": res["gpu_launches"], "clocks": res["clocks"]}
        for k in ("per_op_gbs", "matmul_incr_4096_tflops", "parity_checked", "latency_us_per_batch"):
            if k in res:
                line[k] = res[k]
        if ctx.world == 1 and not args.no_cpu and not args.profile:
            line["cpu_baseline"] = cpu_leg(args.workload, 3 if args.workload == "elementwise" else 1, 1)
            line["cpu_baseline"].pop("ms_per_step", None)
        else:
            line["cpu_baseline"] = None
        if others:
            line["other_workloads"] = others
        print(json.dumps(line), flush=True)
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="yolo",
                    choices=["yolo", "lenet", "mlp", "elementwise", "gemm", "linalg", "backward"])
    ap.add_argument("--elements", type=int, default=1 << 29)
    ap.add_argument("--batch", type=int, default=0,
                    help="global batch of the chosen inference graph instead of the config's (to look at one "
                         "GPU's shard of a multi-GPU run on a single GPU)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-others", action="store_true", help="measure only the chosen workload")
    ap.add_argument("--no-pairs", action="store_true",
                    help="tensor-core kernels never pair CTAs up on 256-row tiles (for comparisons)")
    ap.add_argument("--profile", action="store_true",
                    help="only warm-up and the device-resident timed steps (for runs under a profiler)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        run_ours(args)


if __name__ == "__main__":
    main()

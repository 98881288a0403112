#!/usr/bin/env python
"""Benchmark of the B200 engine on gorgonia's hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line (rank 0). Workloads:
  elementwise  the float32 elementwise/broadcast/fused-chain sweep on vectors of 2^29 elements
               (default; metric GB/s of algorithmic bytes). One step = Add, Mul, Sub, Div, Pow,
               Gt (12 B/elem each), Exp, Tanh, Sigmoid (8 B/elem), broadcast Add of
               (B,1024)+(1,1024) (8 B/elem) and the fused chain tanh(x*w+b) (16 B/elem).

`value` is measured with the inputs resident in HBM; `e2e` is the same step driven through
the C ABI from host buffers: pinned host -> device copies of the step's inputs and a device
-> host read of the step's last result inside the timed region.

With --impl reference the same step runs on the host cores through the CPU oracle (the
restatement of gorgonia's CPU engine; the Go reference itself cannot be built here), on a
bounded sample of the workload.
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


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


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
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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
        # the busiest half of the samples stands for "under load"
        load = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------
# elementwise sweep
# ------------------------------------------------------------------------------------------

def make_inputs(n, seed=2024):
    """x, y ~ N(0,1); base = |x| + 0.1 for Pow; w, b rows of 1024 for the broadcast forms."""
    g = np.random.Generator(np.random.Philox(seed))
    x = g.standard_normal(n, dtype=np.float32)
    y = g.standard_normal(n, dtype=np.float32)
    row = g.standard_normal(1024, dtype=np.float32)
    return x, y, row


def gpu_sweep_step(e, T, n):
    """One step of the sweep on device-resident tensors: 11 engine calls, flushed per op so that
    every op is its own kernel except the chain, which is the point of that entry."""
    x, y, base, row, r = T["x"], T["y"], T["base"], T["row"], T["r"]
    e.Add(x, y, reuse=r); e.DoWork()
    e.Mul(x, y, reuse=r); e.DoWork()
    e.Sub(x, y, reuse=r); e.DoWork()
    e.Div(x, y, reuse=r); e.DoWork()
    e.Pow(base, y, reuse=r); e.DoWork()
    e.Gt(x, y, reuse=r); e.DoWork()
    e.Unary("exp", x, reuse=r); e.DoWork()
    e.Unary("tanh", x, reuse=r); e.DoWork()
    e.Unary("sigmoid", x, reuse=r); e.DoWork()
    e.BroadcastBinary("add", x, row, 1, 1024, reuse=r); e.DoWork()
    # tanh(x*w+b) with full-size w, b: three engine calls, one kernel
    e.Mul(x, y, reuse=r)
    e.Add(r, base, unsafe=True)
    e.Unary("tanh", r, unsafe=True)
    e.DoWork()


def cpu_sweep_step(oracle, x, y, base, row):
    oracle.binary("add", x, y); oracle.binary("mul", x, y); oracle.binary("sub", x, y)
    oracle.binary("div", x, y); oracle.binary("pow", base, y); oracle.binary("gt", x, y)
    oracle.unary("exp", x); oracle.unary("tanh", x); oracle.unary("sigmoid", x)
    oracle.binary_bcast("add", x, row, 1, 1024)
    return oracle.unary("tanh", oracle.binary("add", oracle.binary("mul", x, y), base))


def time_cpu(n_sample, steps, warmup):
    from oracle import oracle
    x, y, row = make_inputs(n_sample)
    base = (np.abs(x) + np.float32(0.1)).astype(np.float32)
    for _ in range(warmup):
        cpu_sweep_step(oracle, x, y, base, row)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_sweep_step(oracle, x, y, base, row)
    dt = (time.perf_counter() - t0) / steps
    return BYTES_PER_ELEM_STEP * n_sample / dt / 1e9, dt, oracle.threads()


def run_reference(args, rank, world):
    if rank != 0:
        return
    n_sample = 1 << 24
    gbs, dt, cores = time_cpu(n_sample, args.steps, min(args.warmup, 1))
    sample = f"{args.steps} steps of the same 11-op sweep on vectors of 2^24 float32 elements"
    line = {
        "impl": "reference", "metric": "elementwise sweep throughput (algorithmic bytes)", "value": gbs,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "elementwise_sweep_f32", "elements": n_sample, "full_workload_elements": 1 << 29},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of gorgonia's CPU-engine semantics (oracle/); the Go reference cannot be built "
                "here (no Go toolchain, dependencies not vendored)",
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank, local_rank, world):
    import torch
    from gorgonia_b200 import Engine

    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    n = args.elements
    e = Engine(device=local_rank, arena_bytes=int(4.25 * 4 * n) + (64 << 20))
    x, y, row = make_inputs(n, seed=2024 + rank)
    base = (np.abs(x) + np.float32(0.1)).astype(np.float32)

    # pinned host copies (the e2e leg copies from these every step)
    def pinned(a):
        p = e.host_alloc(a.nbytes)
        v = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=a.shape)
        v[...] = a
        return p, v

    hx, _ = pinned(x)
    hy, _ = pinned(y)
    hb, _ = pinned(base)
    hout_p = e.host_alloc(4 * n)
    T = {"x": e.empty(n), "y": e.empty(n), "base": e.empty(n), "r": e.empty(n), "row": e.tensor(row)}
    from gorgonia_b200._lib import lib, check
    for t, hp in ((T["x"], hx), (T["y"], hy), (T["base"], hb)):
        check(lib.b200_memcpy_h2d(e.h, t.ptr, hp, 4 * n), e.h)
    del x, y, base

    def barrier():
        e.Signal()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if dist is None:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ev0, ev1 = e.event(), e.event()

    # ---- device-resident leg: `value`
    for _ in range(args.warmup):
        gpu_sweep_step(e, T, n)
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    l0 = e.launches
    e.record(ev0)
    for _ in range(args.steps):
        gpu_sweep_step(e, T, n)
    e.record(ev1)
    barrier()
    ms = max_over_ranks(e.elapsed_ms(ev0, ev1))
    launches = e.launches - l0
    clocks = sampler.stop() if rank == 0 else None
    step_s = ms / 1e3 / args.steps
    bytes_step = BYTES_PER_ELEM_STEP * n
    value = world * bytes_step / step_s / 1e9

    # ---- per-op breakdown (untimed for the headline; each op bracketed by its own events)
    per_op = {}
    if rank == 0 and not args.profile:
        evs = [e.event() for _ in range(2)]
        x_, y_, b_, row_, r_ = T["x"], T["y"], T["base"], T["row"], T["r"]
        ops = {
            "add": lambda: e.Add(x_, y_, reuse=r_), "mul": lambda: e.Mul(x_, y_, reuse=r_),
            "sub": lambda: e.Sub(x_, y_, reuse=r_), "div": lambda: e.Div(x_, y_, reuse=r_),
            "pow": lambda: e.Pow(b_, y_, reuse=r_), "gt": lambda: e.Gt(x_, y_, reuse=r_),
            "exp": lambda: e.Unary("exp", x_, reuse=r_), "tanh": lambda: e.Unary("tanh", x_, reuse=r_),
            "sigmoid": lambda: e.Unary("sigmoid", x_, reuse=r_),
            "bcast_add": lambda: e.BroadcastBinary("add", x_, row_, 1, 1024, reuse=r_),
            "chain_tanh_xw_b": lambda: (e.Mul(x_, y_, reuse=r_), e.Add(r_, b_, unsafe=True),
                                        e.Unary("tanh", r_, unsafe=True)),
        }
        reps = 5
        for name, _, bpe in ELEMENTWISE_OPS:
            ops[name](); e.DoWork()
            e.record(evs[0])
            for _ in range(reps):
                ops[name](); e.DoWork()
            e.record(evs[1])
            t = e.elapsed_ms(evs[0], evs[1]) / reps / 1e3
            per_op[name] = round(bpe * n / t / 1e9, 1)

    # ---- end-to-end leg: host buffers in, host result out, copies inside the timed region
    def e2e_step():
        check(lib.b200_memcpy_h2d_async(e.h, T["x"].ptr, hx, 4 * n), e.h)
        check(lib.b200_memcpy_h2d_async(e.h, T["y"].ptr, hy, 4 * n), e.h)
        check(lib.b200_memcpy_h2d_async(e.h, T["base"].ptr, hb, 4 * n), e.h)
        gpu_sweep_step(e, T, n)
        check(lib.b200_memcpy_d2h_async(e.h, hout_p, T["r"].ptr, 4 * n), e.h)

    e2e_steps = max(2, min(args.steps, 5))
    e2e_value = None
    if not args.profile:
        e2e_step()
        barrier()
        e.record(ev0)
        for _ in range(e2e_steps):
            e2e_step()
        e.record(ev1)
        barrier()
        e2e_ms = max_over_ranks(e.elapsed_ms(ev0, ev1))
        e2e_value = world * bytes_step / (e2e_ms / 1e3 / e2e_steps) / 1e9

    if rank == 0:
        pk = peaks()
        kernel_s = step_s / len(ELEMENTWISE_OPS)      # 11 launches per step, back to back
        achieved = bytes_step / len(ELEMENTWISE_OPS) / kernel_s / 1e9
        cpu = None
        if world == 1 and not args.no_cpu and not args.profile:
            gbs, dt, cores = time_cpu(1 << 24, 3, 1)
            cpu = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                   "sample": "3 steps of the same 11-op sweep on vectors of 2^24 float32 elements"}
        line = {
            "metric": "elementwise sweep throughput (algorithmic bytes)", "value": value, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "elementwise_sweep_f32", "elements": n, "ops": [o for o, _, _ in ELEMENTWISE_OPS],
                       "bytes_per_element_step": BYTES_PER_ELEM_STEP, "l2": "inputs larger than L2",
                       "parallelism": f"replicas x{world}" if world > 1 else "single GPU"},
            "roofline": {"bound": "hbm", "kernel": "pw_kernel", "achieved": achieved, "peak": pk["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "peak_source": pk["source"],
                         "frac_of_nominal_8TBs": achieved / 8000.0, "traffic": None},
            "per_op_gbs": per_op,
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 3 * 4 * n,
                    "d2h_bytes_per_step": 4 * n, "steps": e2e_steps},
            "gpu_launches": launches,
            "clocks": clocks,
            "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    e.Close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="elementwise", choices=["elementwise"])
    ap.add_argument("--elements", type=int, default=1 << 29)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--profile", action="store_true",
                    help="only warm-up and the device-resident timed steps (for runs under a profiler)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()

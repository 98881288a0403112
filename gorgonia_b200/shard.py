"""Batch sharding of an inference tape over the GPUs of one box.

Samples are independent, weights are replicated, so the forward path needs no collective: rank r
runs the same tape on the contiguous slice shard_bounds(total, world)[r] of the batch and writes
its rows of the result. The only things that cross ranks are the rendezvous and the reduction of
the timings (max over ranks), both through torch.distributed; gorgonia itself has nothing to
mirror here (its VM drives device 0 only: analysis.go:52-65).
"""


def shard_bounds(total, world):
    """Contiguous [start, stop) per rank; the first (total % world) ranks get one extra sample."""
    if world <= 0 or total < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(total, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((start, start + n))
        start += n
    return out


def my_shard(total, rank, world):
    return shard_bounds(total, world)[rank]


def max_over_ranks(value, dist=None, device=None):
    """The slowest rank's figure: what a whole-job time is. dist = torch.distributed or None."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def all_gather_rows(local_rows, total, dist=None):
    """Concatenates every rank's rows (numpy, shape (n_r, ...)) in rank order; used by tests and by
    callers that want the whole result on every rank. The benchmark does not need it."""
    import numpy as np
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return local_rows
    import torch
    world = dist.get_world_size()
    bounds = shard_bounds(total, world)
    width = max(b - a for a, b in bounds)
    pad = np.zeros((width,) + local_rows.shape[1:], dtype=local_rows.dtype)
    pad[:local_rows.shape[0]] = local_rows
    mine = torch.from_numpy(pad)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    return np.concatenate([p.numpy()[:b - a] for p, (a, b) in zip(parts, bounds)], axis=0)


class Comm:
    """The training variant's communicator over the C ABI (b200_comm_*): a transport function behind
    a pointer plus rank and world size. Comm.nccl binds NCCL for an engine's device; Comm.from_callable
    wraps any Python all-reduce (CPU ranks over gloo in the tests)."""

    def __init__(self, handle, keep=None):
        self.h = handle
        self._keep = keep          # the ctypes callback must outlive the communicator

    @classmethod
    def from_callable(cls, allreduce, rank, world):
        """allreduce(array) sums a numpy array over the ranks in place; it may raise or return a
        non-zero code to report a failure."""
        import ctypes as C

        import numpy as np

        from . import _lib

        def transport(_ctx, buf, count, dtype, _stream):
            try:
                ct = C.c_float if dtype == _lib.F32 else C.c_double
                view = np.ctypeslib.as_array(C.cast(buf, C.POINTER(ct)), shape=(count,))
                rc = allreduce(view)
                return int(rc or 0)
            except Exception:      # noqa: BLE001 - an exception must not unwind through C
                return -1

        cb = _lib.ALLREDUCE_FN(transport)
        h = C.c_void_p()
        rc = _lib.lib.b200_comm_create(cb, None, rank, world, C.byref(h))
        if rc != _lib.OK:
            raise _lib.B200Error(rc, "b200_comm_create: bad rank or world size")
        return cls(h, keep=cb)

    @classmethod
    def nccl(cls, engine, dist):
        """NCCL communicator for the engine's device; the 128-byte id travels from rank 0 to the
        others through the process group the caller already has (torch.distributed)."""
        import ctypes as C

        import torch

        from . import _lib
        rank, world = dist.get_rank(), dist.get_world_size()
        uid = (C.c_ubyte * 128)()
        if rank == 0:
            _lib.check(_lib.lib.b200_nccl_unique_id(uid))
        t = torch.tensor(list(uid), dtype=torch.uint8, device=f"cuda:{engine.device}")
        dist.broadcast(t, 0)
        raw = bytes(t.cpu().tolist())
        buf = (C.c_ubyte * 128).from_buffer_copy(raw)
        h = C.c_void_p()
        _lib.check(_lib.lib.b200_comm_create_nccl(engine.h, buf, rank, world, C.byref(h)), engine.h)
        return cls(h)

    @property
    def world(self):
        from . import _lib
        return _lib.lib.b200_comm_world(self.h)

    def allreduce_mean_(self, tensor):
        """Averages an engine Tensor (device) or a numpy array (host, CPU ranks) over the ranks, in place."""
        import numpy as np

        from . import _lib
        if isinstance(tensor, np.ndarray):
            code = _lib.F32 if tensor.dtype == np.float32 else _lib.F64
            rc = _lib.lib.b200_comm_allreduce_mean_host(self.h, tensor.ctypes.data, tensor.size, code)
            if rc != _lib.OK:
                raise _lib.B200Error(rc, (_lib.lib.b200_comm_last_error(self.h) or b"").decode())
            return tensor
        from .engine import dtype_code
        e = tensor.engine
        _lib.check(_lib.lib.b200_allreduce_mean(e.h, self.h, tensor.ptr, tensor.size, dtype_code(tensor.dtype)), e.h)
        return tensor

    def close(self):
        from . import _lib
        if self.h:
            _lib.lib.b200_comm_destroy(self.h)
            self.h = None


def allreduce_mean_(tensor, dist, engine=None, comm=None):
    """Training variant only: averages a flat gradient bucket over the ranks, in place.

    gorgonia has no distributed path; its data-parallel precedent applies the gradients of several
    VMs serially through one solver (example_concurrent_training_test.go:80-115). Here every rank
    holds a replica, and after the last backward kernel one all-reduce (sum) over NVLink runs on the
    flat bucket, followed by a scale by 1/world on the engine, before Solver.Step. One bucket,
    because the buckets of these models are small (LeNet: 818 698 floats) and latency bound.
    `tensor` is an engine Tensor (float32 or float64): NCCL through b200_allreduce_mean; or, with
    gloo (CPU tests), a numpy array summed by torch.distributed through the same C entry points.
    Pass `comm` to reuse a communicator; otherwise one is made and closed. The forward path never
    calls this.
    """
    import numpy as np
    world = dist.get_world_size() if dist is not None and dist.is_initialized() else 1
    if world == 1:
        return tensor
    own = comm is None
    if isinstance(tensor, np.ndarray):
        if own:
            import torch

            def gloo_sum(view):
                dist.all_reduce(torch.from_numpy(view), op=dist.ReduceOp.SUM)
                return 0
            comm = Comm.from_callable(gloo_sum, dist.get_rank(), world)
    elif own:
        comm = Comm.nccl(engine or tensor.engine, dist)
    try:
        return comm.allreduce_mean_(tensor)
    finally:
        if own:
            comm.close()

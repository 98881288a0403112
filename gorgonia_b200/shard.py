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


class _DevicePtr:
    """Exposes a range of engine memory through __cuda_array_interface__ so that torch can wrap it
    without copying."""

    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (int(n),), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2}


def allreduce_mean_(tensor, dist, engine=None):
    """Training variant only: averages a flat gradient bucket over the ranks, in place.

    gorgonia has no distributed path; its data-parallel precedent applies the gradients of several
    VMs serially through one solver (example_concurrent_training_test.go:80-115). Here every rank
    holds a replica, and after the last backward kernel one NCCL all-reduce (sum) over NVLink runs
    on the flat bucket, followed by a scale by 1/world on the engine, before Solver.Step. One
    bucket, because the buckets of these models are small (LeNet: 818 698 floats) and latency
    bound. `tensor` is an engine Tensor (float32 or float64); with gloo (CPU tests) a numpy array.
    The forward path never calls this.
    """
    import numpy as np
    import torch
    world = dist.get_world_size() if dist is not None and dist.is_initialized() else 1
    if isinstance(tensor, np.ndarray):                       # CPU ranks (gloo): the same arithmetic
        if world > 1:
            t = torch.from_numpy(tensor)
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            tensor /= tensor.dtype.type(world)
        return tensor
    if world == 1:
        return tensor
    engine = engine or tensor.engine
    engine.Signal()                                          # the bucket is complete on the device
    typestr = "<f4" if tensor.dtype == np.float32 else "<f8"
    with torch.cuda.device(engine.device):
        view = torch.as_tensor(_DevicePtr(tensor.ptr, tensor.size, typestr), device=f"cuda:{engine.device}")
        dist.all_reduce(view, op=dist.ReduceOp.SUM)
        torch.cuda.synchronize()
    engine.DivScalar(tensor, float(world), unsafe=True)      # sum / world, as the solver expects a mean
    return tensor

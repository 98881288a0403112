"""Two-GPU checks (skipped when the box has one GPU): the batch-sharded forward equals the single-GPU
forward (bit for bit when no tile's k range is shared between CTAs, which is a function of the batch
size; within the GEMM tolerance otherwise), and the training-variant gradient all-reduce averages
over NCCL.

Each rank is a child process with its own engine; a rank leaves only between steps, with nothing
in flight; NVLS is off (plain NCCL rings), as the pool's rules for multi-process GPU tests ask."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from gorgonia_b200 import Engine, shard, tapes
        total = 48
        x = np.random.Generator(np.random.Philox(3)).random((total, 1, 28, 28), dtype=np.float32)
        a, b = shard.my_shard(total, rank, world)
        fixed = Engine(rank, 1 << 30, streamk=False)     # one summation order whatever the batch size
        m = tapes.LeNet(fixed, b - a)
        m.x.set(x[a:b])
        local_fixed = m.forward().numpy()
        fixed.Close()
        e = Engine(rank, 1 << 30)
        m = tapes.LeNet(e, b - a)
        m.x.set(x[a:b])
        local = m.forward().numpy()
        grad = e.tensor(np.full(100_000, float(rank + 1), np.float32))
        shard.allreduce_mean_(grad, dist)
        g = grad.numpy()
        dist.barrier()
        q.put((rank, a, b, local_fixed, local, float(g.min()), float(g.max())))
        e.Close()
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharded_forward_and_gradient_allreduce():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted([q.get(timeout=300) for _ in range(2)])
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    from gorgonia_b200 import Engine, tapes
    from tests.util import assert_gemm_close
    x = np.random.Generator(np.random.Philox(3)).random((48, 1, 28, 28), dtype=np.float32)
    want = {}
    for streamk in (False, True):
        e = Engine(0, 1 << 30, streamk=streamk)
        m = tapes.LeNet(e, 48)
        m.x.set(x)
        want[streamk] = m.forward().numpy()
        e.Close()
    for rank, a, b, local_fixed, local, gmin, gmax in got:
        assert np.array_equal(local_fixed, want[False][a:b])   # sharding changes nothing, bit for bit
        assert_gemm_close(local, want[True][a:b], 1e-5)
        assert gmin == gmax == 1.5

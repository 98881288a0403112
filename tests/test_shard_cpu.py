"""The multi-rank path on CPU: two gloo ranks shard a batch, run the graph on their slices (with the
CPU oracle standing in for the device) and the pieces reassemble to the single-rank result; the
timing reduction takes the slowest rank."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gorgonia_b200 import shard


def test_shard_bounds_partition_the_batch():
    for total in (0, 1, 7, 64, 256, 8192):
        for world in (1, 2, 3, 4, 8):
            b = shard.shard_bounds(total, world)
            assert b[0][0] == 0 and b[-1][1] == total
            assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
            sizes = [y - x for x, y in b]
            assert max(sizes) - min(sizes) <= 1
    assert shard.shard_bounds(8192, 8) == [(i * 1024, (i + 1) * 1024) for i in range(8)]
    with pytest.raises(ValueError):
        shard.shard_bounds(4, 0)


class _HostLeNet:
    pass


def _host_lenet():
    from gorgonia_b200 import tapes
    g = np.random.Generator(np.random.Philox(5))
    h, ch = _HostLeNet(), tapes.LeNet.CH
    h.wc_host = [tapes.he_normal(g, (ch[i + 1], ch[i], 3, 3), ch[i] * 9) for i in range(3)]
    h.wd_host = [tapes.he_normal(g, (1152, 625), 1152), tapes.he_normal(g, (625, 10), 625)]
    return h


def _worker(rank, world, port, total, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import graphs
        model = _host_lenet()                       # replicated weights: same seed on every rank
        x = np.random.Generator(np.random.Philox(11)).random((total, 1, 28, 28), dtype=np.float32)
        a, b = shard.my_shard(total, rank, world)
        local = graphs.lenet(model, x[a:b])
        whole = shard.all_gather_rows(local, total, dist)
        slowest = shard.max_over_ranks(10.0 + rank, dist)
        grad = np.full(1000, float(rank + 1), np.float32)     # ranks hold 1s and 2s: the mean is 1.5
        shard.allreduce_mean_(grad, dist)                      # through b200_comm_* with a gloo transport
        assert np.all(grad == np.float32(1.5))
        _comm_error_paths(rank, world)
        dist.barrier()
        if rank == 0:
            q.put((whole, slowest))
    finally:
        dist.destroy_process_group()


def _comm_error_paths(rank, world):
    """Failures are made on the host: a transport that reports an error code on one rank after the
    exchange took place, and one that raises. The failing rank gets B200_ERR_CUDA and an unscaled
    bucket, the other rank its mean; nobody hangs because every rank still takes part in the exchange."""
    from gorgonia_b200 import _lib
    from gorgonia_b200._lib import B200Error

    def summed(view):
        dist.all_reduce(torch.from_numpy(view), op=dist.ReduceOp.SUM)

    def fails_on_rank_1(view):
        summed(view)
        return 7 if rank == 1 else 0

    def raises_on_rank_0(view):
        summed(view)
        if rank == 0:
            raise RuntimeError("link down")

    for transport, bad_rank in ((fails_on_rank_1, 1), (raises_on_rank_0, 0)):
        comm = shard.Comm.from_callable(transport, rank, world)
        assert comm.world == world
        g = np.full(64, float(rank + 1), np.float64)
        if rank == bad_rank:
            with pytest.raises(B200Error) as ei:
                comm.allreduce_mean_(g)
            assert ei.value.code == _lib.ERR_CUDA and "not a mean" in str(ei.value)
            assert np.all(g == 3.0)                          # summed by the transport, not divided
        else:
            comm.allreduce_mean_(g)
            assert np.all(g == 1.5)
        # the communicator stays usable after a failure
        comm.close()
    ok = shard.Comm.from_callable(lambda v: summed(v), rank, world)
    g = np.arange(8, dtype=np.float32) * (rank + 1)
    ok.allreduce_mean_(g)
    assert np.array_equal(g, np.arange(8, dtype=np.float32) * 1.5)
    empty = np.zeros(0, np.float32)
    ok.allreduce_mean_(empty)                                # nothing to do, no exchange
    ok.close()
    with pytest.raises(B200Error):
        shard.Comm.from_callable(summed, 5, world)           # rank outside the world


def test_two_ranks_reassemble_the_single_rank_result():
    total, world = 9, 2                              # uneven on purpose: shards of 5 and 4
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, world, port, total, q)) for r in range(world)]
    for p in procs:
        p.start()
    whole, slowest = q.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    from oracle import graphs
    x = np.random.Generator(np.random.Philox(11)).random((total, 1, 28, 28), dtype=np.float32)
    want = graphs.lenet(_host_lenet(), x)
    assert whole.shape == want.shape
    assert np.array_equal(whole, want)               # samples are independent: sharding changes nothing
    assert slowest == 11.0

"""Host-side logic of the data-parallel path on CPU ranks (gloo, world size 2): row sharding, bucket
tiling, asynchronous bucketed all-reduce of a flat gradient buffer, the lr/world update rule, and
failure detection by a short process-group timeout when a rank never joins a collective."""
import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mcw_cppamp_torch_b200 import dp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _init(rank, world, port, timeout_s=60):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _grad(X, y, w):
    """Mean-squared-error gradient of a linear model on a batch: the per-rank 'backward'."""
    r = X @ w - y
    return (2.0 / len(y)) * (X.T @ r)


def _worker_allreduce(rank, world, port, out):
    _init(rank, world, port)
    rs = np.random.RandomState(0)
    B, D = 16, 10
    X, y, w = rs.standard_normal((B, D)), rs.standard_normal(B), rs.standard_normal(D)
    lo, hi = dp.shard_rows(B, rank, world)
    flat = torch.from_numpy(_grad(X[lo:hi], y[lo:hi], w).copy())
    buckets = dp.GradBuckets(flat, [(6, D), (0, 6)])       # the tail bucket becomes ready first
    buckets.launch(0)
    buckets.launch(1)
    buckets.wait()
    # sums of per-rank batch means; dividing the step by the world size gives the global mean
    lr = 0.1
    w_dp = w - (lr / world) * flat.numpy()
    w_full = w - lr * _grad(X, y, w)
    out.put((rank, float(np.abs(w_dp - w_full).max())))
    dist.destroy_process_group()


def test_bucketed_allreduce_equals_full_batch_gradient():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_allreduce, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == [0, 1]
    assert all(err < 1e-12 for _, err in res)


def test_shard_rows_and_bucket_validation():
    assert [dp.shard_rows(1024, r, 8) for r in (0, 7)] == [(0, 128), (896, 1024)]
    with pytest.raises(ValueError):
        dp.shard_rows(10, 0, 4)
    flat = torch.zeros(10)
    dp.GradBuckets(flat, [(4, 10), (0, 4)])
    for bad in ([(0, 4), (5, 10)], [(0, 4), (4, 9)], [(0, 11)], [(3, 3), (0, 10)]):
        with pytest.raises(ValueError):
            dp.GradBuckets(flat, bad)
    # single process: launching is a no-op, nothing pends
    b = dp.GradBuckets(flat, [(0, 10)])
    b.launch(0)
    b.wait()
    assert dp.world() == (0, 1)


def _worker_missing_peer(rank, world, port, out):
    _init(rank, world, port, timeout_s=3)
    t = torch.ones(4)
    def report(msg):
        out.put((rank, msg))
        out.close()
        out.join_thread()       # flush before the hard exit below
        os._exit(0)
    if rank == 1:
        # this rank leaves between steps without joining the collective (a host-side failure)
        report("left")
    try:
        dist.all_reduce(t)
        report("no error")
    except Exception as e:      # the survivor learns of it through the process-group timeout / closed peer
        report("detected: " + type(e).__name__)


def test_a_rank_that_never_joins_is_detected_by_timeout():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_missing_peer, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(60)
    assert res[1] == "left"
    assert res[0].startswith("detected"), res

"""Host-side logic of the data-parallel path on CPU: THGPUComm's bucket table, launch order, cross-rank layout
check and watchdog, driven through transport callbacks the tests control -- first a fake transport in one process
(failures injected on the host: a bucket that never completes, a transport error), then two gloo ranks whose
callbacks move the flat gradient buffer (host memory here) through torch.distributed.  No GPU is involved: the
library only passes the buffer's address through to the callbacks."""
import ctypes as C
import datetime
import os
import socket
import time

import numpy as np
import pytest

from mcw_cppamp_torch_b200 import GPUTensor, THCError, dp, lib


def host_tensor(a):
    """A THGPUTensor whose storage borrows the memory of numpy array `a` (never dereferenced by the library here)."""
    L = lib()
    st = L.THGPUStorage_newWithData(C.c_void_p(a.ctypes.data), a.size)
    t = GPUTensor(_ptr=L.THGPUTensor_newWithStorage1d(st, 0, a.size, 1))
    L.THGPUStorage_free(st)
    return t


def view(ptr, count):
    return np.ctypeslib.as_array((C.c_float * count).from_address(ptr))


class FakeTransport:
    """Single-process transport: records what was queued; `pending` buckets never complete, `broken` ones report an error."""

    def __init__(self, same_layout=1):
        self.queued, self.aborted, self.same_layout = [], 0, same_layout
        self.pending, self.broken, self.update = set(), set(), None

    def callbacks(self):
        def all_reduce(ctx, bucket, data, begin, count):
            self.queued.append((bucket, begin, count))
            view(data, count)[:] *= 2.0                     # "sum over two identical ranks"
            if self.update:
                w, lr = self.update
                w[begin:begin + count] -= lr * view(data, count)
            return 0

        def set_update(ctx, w, v, lr, momentum):
            self.update = (self.w_host, lr)
            return 0

        def done(ctx, bucket):
            return -1 if bucket in self.broken else 0 if bucket in self.pending else 1

        def agree(ctx, values, n):
            self.signature = [values[i] for i in range(n)]
            return self.same_layout

        def abort(ctx):
            self.aborted += 1
            return 0
        return dict(all_reduce=all_reduce, set_update=set_update, done=done, join=lambda ctx: 0, agree=agree, abort=abort)


def test_bucket_table_launch_order_and_update():
    tr = FakeTransport()
    comm = dp.Comm.with_backend(2, 0, **tr.callbacks())
    g = np.arange(10, dtype=np.float32)
    w = np.ones(10, np.float32)
    tr.w_host = w
    fg, fw = host_tensor(g), host_tensor(w)
    with pytest.raises(THCError, match="set the gradient buckets first"):
        comm.launch(0)
    for bad, msg in (([(0, 4), (3, 10)], "overlap"), ([(0, 11)], "outside"), ([(4, 4), (0, 10)], "outside")):
        with pytest.raises(THCError, match=msg):
            comm.set_buckets(fg, bad)
    comm.set_buckets(fg, [(6, 10), (0, 6)])                 # the tail bucket becomes ready first
    assert tr.signature == [10, 2, 6, 10, 0, 6]             # what every rank must agree on
    comm.set_update(fw, None, 0.5, 0.0)
    comm.launch(0)
    with pytest.raises(THCError, match="already queued"):
        comm.launch(0)
    with pytest.raises(THCError, match="never queued"):
        comm.wait()
    with pytest.raises(THCError, match="no such bucket"):
        comm.launch(2)
    comm.launch(1)
    comm.wait()
    assert tr.queued == [(0, 6, 4), (1, 0, 6)]
    assert np.array_equal(g, 2 * np.arange(10)) and np.array_equal(w, 1 - 0.5 * g)
    comm.launch(0); comm.launch(1); comm.wait()             # the next step may queue every bucket again
    assert comm.error() is None and tr.aborted == 0
    comm.close()


def test_layout_mismatch_is_refused_before_anything_is_queued():
    tr = FakeTransport(same_layout=0)
    comm = dp.Comm.with_backend(2, 1, **tr.callbacks())
    g = np.zeros(8, np.float32)
    with pytest.raises(THCError, match="layout differs between ranks.*nothing was queued"):
        comm.set_buckets(host_tensor(g), [(0, 8)])
    assert tr.queued == []
    with pytest.raises(THCError, match="set the gradient buckets first"):
        comm.launch(0)
    comm.close()


@pytest.mark.parametrize("kind", ["timeout", "transport_error"])
def test_watchdog_aborts_a_bucket_that_does_not_complete(kind):
    tr = FakeTransport()
    comm = dp.Comm.with_backend(2, 0, **tr.callbacks())
    g = np.zeros(8, np.float32)
    comm.set_buckets(host_tensor(g), [(4, 8), (0, 4)])
    comm.set_timeout(0.2)
    (tr.pending if kind == "timeout" else tr.broken).add(1)  # bucket 1's all-reduce never completes / fails
    comm.launch(0)
    comm.launch(1)
    comm.wait()                                             # queues the join; does not block on the host
    t0 = time.time()
    while comm.error() is None and time.time() - t0 < 5:
        time.sleep(0.01)
    assert comm.error() is not None and tr.aborted == 1
    assert ("did not complete within" if kind == "timeout" else "reported an error") in comm.error()
    assert "bucket 1" in comm.error()
    if kind == "timeout":
        assert time.time() - t0 >= 0.15
    for call in (lambda: comm.launch(0), comm.wait):        # a dead communicator refuses further work with the reason
        with pytest.raises(THCError, match="communicator aborted"):
            call()
    comm.close()


def test_shard_rows_and_layer_buckets():
    assert [dp.shard_rows(1024, r, 8) for r in (0, 7)] == [(0, 128), (896, 1024)]
    with pytest.raises(ValueError):
        dp.shard_rows(10, 0, 4)

    class P:
        def __init__(self, n): self.n = n
        def nElement(self): return self.n

    class M:
        def __init__(self, *sizes): self.sizes = sizes
        def parameters(self): return ([P(k) for k in self.sizes], None) if self.sizes else None

    class Net:
        def modules_list(self): return [M(10, 2), M(), M(30, 3), M(100, 5), M(7, 1)]
    spans, owner = dp.layer_buckets(Net())
    assert spans == [(150, 158), (45, 150), (12, 45), (0, 12)]          # backward order: last module first
    assert owner == {0: (0, True), 1: (1, True), 2: (2, True), 3: (3, True)}
    spans, owner = dp.layer_buckets(Net(), min_elements=100)
    assert spans == [(45, 158), (0, 45)]                                 # 8 + 105 reaches 100; the rest is the last bucket
    assert owner == {0: (0, False), 1: (0, True), 2: (1, False), 3: (1, True)}
    spans, owner = dp.layer_buckets(Net(), min_elements=10 ** 6)
    assert spans == [(0, 158)] and owner[3] == (0, True) and not owner[0][1]


# ---------------------------------------------------------------- two gloo ranks
def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _grad(X, y, w):
    r = X @ w - y
    return ((2.0 / len(y)) * (X.T @ r)).astype(np.float32)


def _gloo_comm(rank, world, state):
    """THGPUComm whose transport is torch.distributed (gloo) on host memory."""
    import torch
    import torch.distributed as dist

    def all_reduce(ctx, bucket, data, begin, count):
        t = torch.from_numpy(view(data, count))
        state["work"][bucket] = (dist.all_reduce(t, op=dist.ReduceOp.SUM, async_op=True), begin, count, t)
        return 0

    def set_update(ctx, w, v, lr, momentum):
        state["lr"] = lr
        return 0

    def done(ctx, bucket):
        item = state["work"].get(bucket)
        if item is None:
            return 0
        work, begin, count, t = item
        if not work.is_completed():
            return 0
        try:
            work.wait()                                      # completed: returns at once, or raises what went wrong
        except Exception:
            return -1
        return 1

    def join(ctx):                                           # host transport: joining means waiting
        for bucket, (work, begin, count, t) in list(state["work"].items()):
            try:
                work.wait()
            except Exception:
                return 1
            if "lr" in state:
                state["w"][begin:begin + count] -= state["lr"] * t.numpy()
        return 0

    def agree(ctx, values, n):
        v = torch.tensor([values[i] for i in range(n)], dtype=torch.int64)
        hi, lo = v.clone(), v.clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        return int(bool((hi == lo).all()))

    def abort(ctx):
        state["aborted"] = True
        return 0
    return dp.Comm.with_backend(world, rank, all_reduce=all_reduce, set_update=set_update, done=done, join=join,
                                agree=agree, abort=abort)


def _init(rank, world, port, timeout_s=60):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _worker_step(rank, world, port, out):
    import torch.distributed as dist
    _init(rank, world, port)
    rs = np.random.RandomState(0)
    B, D = 16, 10
    X, y, w0 = rs.standard_normal((B, D)), rs.standard_normal(B), rs.standard_normal(D).astype(np.float32)
    lo, hi = dp.shard_rows(B, rank, world)
    g = _grad(X[lo:hi], y[lo:hi], w0)
    w = w0.copy()
    state = {"work": {}, "w": w}
    comm = _gloo_comm(rank, world, state)
    fg, fw = host_tensor(g), host_tensor(w)
    # a layout that differs on one rank is refused on both before any gradient moves
    try:
        comm.set_buckets(fg, [(6, D), (0, 6)] if rank == 0 else [(5, D), (0, 5)])
        mismatch = "accepted"
    except THCError as e:
        mismatch = "refused" if "layout differs" in str(e) else str(e)
    comm.set_buckets(fg, [(6, D), (0, 6)])
    lr = 0.1
    comm.set_update(fw, None, lr / world, 0.0)              # sums of per-rank batch means: lr / world is the global mean
    comm.launch(0)
    comm.launch(1)
    comm.wait()
    w_full = w0 - lr * _grad(X, y, w0)
    out.put((rank, mismatch, float(np.abs(w - w_full).max()), comm.error()))
    comm.close()
    dist.destroy_process_group()


def _run(target, world=2, timeout_s=120):
    import torch.multiprocessing as mp
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=target, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=timeout_s) for _ in range(world)]
    for p in procs:
        p.join(60)
    return res, procs


def test_two_ranks_bucketed_allreduce_and_update_equal_the_full_batch_step():
    res, procs = _run(_worker_step)
    assert all(p.exitcode == 0 for p in procs)
    assert sorted(r[0] for r in res) == [0, 1]
    for rank, mismatch, err, comm_error in res:
        assert mismatch == "refused" and err < 1e-6 and comm_error is None


def _worker_missing_peer(rank, world, port, out):
    _init(rank, world, port, timeout_s=30)

    def report(msg):
        out.put((rank, msg))
        out.close()
        out.join_thread()       # flush before the hard exit below
        os._exit(0)
    g = np.ones(8, np.float32)
    state = {"work": {}, "w": np.zeros(8, np.float32)}
    comm = _gloo_comm(rank, world, state)
    comm.set_buckets(host_tensor(g), [(0, 8)])
    comm.set_timeout(1.0)
    if rank == 1:
        report("left")          # this rank leaves between steps without joining the collective (a host-side failure)
    comm.launch(0)
    t0 = time.time()
    while comm.error() is None and time.time() - t0 < 20:
        time.sleep(0.02)
    report("detected: %s (aborted=%s)" % (comm.error(), state.get("aborted")))


def test_a_rank_that_never_joins_is_detected_by_the_watchdog():
    res, procs = _run(_worker_missing_peer)
    res = dict(res)
    assert res[1] == "left"
    # gloo either never completes the collective (watchdog deadline) or fails it once the peer's socket closes
    assert res[0].startswith(("detected: all-reduce of gradient bucket 0 did not complete",
                              "detected: the transport reported an error on gradient bucket 0")), res
    assert "communicator aborted (aborted=True)" in res[0], res

"""THGPUComm over NCCL between two GPUs of one box: two ranks, each with a replica of a small conv + Linear net and
half of the batch, take two SGD steps with the bucketed exchange (per-bucket all-reduce and update on the
communicator's stream, nothing synchronising the host) and must end with the weights one process gets from the
whole batch.  Runs as two child processes, one per GPU; skipped on a box with fewer than two.  No failure is
injected here (the missing-peer and transport-error paths are tested on CPU ranks in tests/test_dp_gloo.py)."""
import os

import numpy as np
import pytest
import torch  # noqa: F401  -- see tests/test_gpu_comm.py: before anything loads the system's NCCL

pytestmark = pytest.mark.gpu

LR, MOM, STEPS, BATCH = 0.05, 0.9, 2, 8


def _build(gt, rng):
    nn = gt.nn
    net = nn.Sequential()
    net.add(nn.SpatialConvolutionMM(32, 64, 3, 3, 1, 1, 1, rng=rng)).add(nn.ReLU()).add(nn.SpatialMaxPooling(2, 2, 2, 2))
    net.add(nn.View(64 * 6 * 6)).add(nn.Linear(64 * 6 * 6, 40, rng=rng)).add(nn.LogSoftMax())
    return net


def _data(oracle):
    g = oracle.port.rng(11)
    x = g.uniform((BATCH, 32, 12, 12), -1, 1)
    y = np.array([1 + (7 * i) % 40 for i in range(BATCH)], np.float32)
    return x, y


def _train(gt, oracle, lo, hi, comm_args):
    """Two steps on rows [lo, hi); comm_args = (world, rank, exchange) or None for one process on the whole batch."""
    from mcw_cppamp_torch_b200 import dp
    L = gt.lib()
    net = _build(gt, oracle.port.rng(5))
    net.gpu()
    crit = gt.nn.ClassNLLCriterion()
    fw, fg = net.getParameters()
    fv = gt.GPUTensor(fw.nElement()).fill(0)
    x, y = _data(oracle)
    xg, yg = gt.gpu(x[lo:hi]), gt.gpu(y[lo:hi])
    world = comm_args[0] if comm_args else 1
    comm = None
    if comm_args:
        comm = dp.Comm.nccl(*comm_args)
        spans, owner = dp.layer_buckets(net)
        comm.set_buckets(fg, spans)
        comm.set_update(fw, fv, LR / world, MOM)      # sums over ranks of per-rank batch means
        mods = [m for m in net.modules_list() if m.parameters()][::-1]
        bucket_of = {id(m): owner[i][0] for i, m in enumerate(mods)}
    for _ in range(STEPS):
        fg.zero()
        out = net.forward(xg)
        crit.updateOutput(out, yg, read_back=False)
        g = crit.updateGradInput(out, yg)
        ms = net.modules
        for i in range(len(ms) - 1, -1, -1):
            g = ms[i].backward(ms[i - 1].output if i > 0 else xg, g, 1.0)
            if comm is not None and id(ms[i]) in bucket_of:
                comm.launch(bucket_of[id(ms[i])])
        if comm is not None:
            comm.wait()
        else:
            L.THGPUNN_SGD_update(fw.cdata, fg.cdata, fv.cdata, LR, MOM)
    w = fw.float()
    err = comm.error() if comm is not None else None
    if comm is not None:
        comm.close()
    return w, err


def _worker(rank, world, to_peer, from_peer, out):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch  # noqa: F401  (its NCCL first, as above)
    import mcw_cppamp_torch_b200 as gt
    import oracle
    gt.lib().THGPUSetDevice(rank)

    def exchange(raw):
        if rank == 0:
            to_peer.put(raw)
            return raw
        return from_peer.get(timeout=120)
    lo, hi = rank * BATCH // world, (rank + 1) * BATCH // world
    w, err = _train(gt, oracle, lo, hi, (world, rank, exchange))
    out.put((rank, w, err))


def test_two_gpus_bucketed_exchange_equals_the_whole_batch_step(oracle_port):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    import mcw_cppamp_torch_b200 as gt
    import oracle
    ctx = mp.get_context("spawn")
    idq, out = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, idq, idq, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict()
    for _ in range(2):
        rank, w, err = out.get(timeout=300)
        res[rank] = (w, err)
    for p in procs:
        p.join(60)
    assert all(p.exitcode == 0 for p in procs)
    gt.lib().THGPUInit()
    want, _ = _train(gt, oracle, 0, BATCH, None)
    assert res[0][1] is None and res[1][1] is None
    assert np.array_equal(res[0][0], res[1][0])                       # the replicas stay identical bit for bit
    np.testing.assert_allclose(res[0][0], want, rtol=1e-4, atol=1e-5)

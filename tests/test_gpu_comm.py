"""THGPUComm over its NCCL transport on one GPU (a communicator of one rank: the all-reduce is the identity, every
stream, event and update step is the real one).  The multi-rank host logic is covered on CPU ranks in
tests/test_dp_gloo.py; here: the bucketed exchange + per-bucket SGD equals the plain SGD update, and the stream
ordering holds with nothing synchronising the host."""
import numpy as np
import pytest
import torch  # noqa: F401  -- before the library loads NCCL: torch bundles a newer libnccl.so.2 than the system's, and
#                              the loader hands whichever copy came first to everyone who asks for that soname later

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gt():
    import mcw_cppamp_torch_b200 as m
    m.lib().THGPUInit()
    return m


def test_bucketed_exchange_and_update_equal_plain_sgd(gt, oracle_port):
    from mcw_cppamp_torch_b200 import dp
    g = oracle_port.rng(3)
    n = 1_000_003
    w0, grad, v0 = g.normal((n,)), g.normal((n,)), g.normal((n,))
    comm = dp.Comm.nccl(1, 0, lambda raw: raw)
    fw, fg, fv = gt.gpu(w0), gt.gpu(grad), gt.gpu(v0)
    bounds = [(700_000, n), (300_001, 700_000), (0, 300_001)]            # odd boundaries: unaligned slices
    comm.set_buckets(fg, bounds)
    comm.set_update(fw, fv, 0.01, 0.9)
    ref_w, ref_v = gt.gpu(w0), gt.gpu(v0)
    L = gt.lib()
    for step in range(3):                                                 # nothing synchronises the host in between
        fg.mul(fg, 0.5)                                                   # "backward" rewrites the gradients ...
        for b in range(3):
            comm.launch(b)                                                # ... each bucket leaves as soon as it is queued
        comm.wait()
        L.THGPUNN_SGD_update(ref_w.cdata, fg.cdata, ref_v.cdata, 0.01, 0.9)
    assert comm.error() is None
    assert np.array_equal(fw.float(), ref_w.float()) and np.array_equal(fv.float(), ref_v.float())
    with pytest.raises(gt.THCError, match="never queued"):
        comm.launch(0); comm.wait()
    comm.close()


def test_plain_sgd_when_momentum_is_zero_and_layout_errors(gt, oracle_port):
    from mcw_cppamp_torch_b200 import dp
    g = oracle_port.rng(4)
    w0, grad = g.normal((4096,)), g.normal((4096,))
    comm = dp.Comm.nccl(1, 0, lambda raw: raw, max_ctas=4)             # THGPUComm_newWithOptions: capped collective
    fw, fg = gt.gpu(w0), gt.gpu(grad)
    with pytest.raises(gt.THCError, match="set the gradient buckets first"):
        comm.set_update(fw, None, 0.1, 0.0)
    comm.set_buckets(fg, [(0, 4096)])
    with pytest.raises(gt.THCError, match="velocity buffer"):
        comm.set_update(fw, None, 0.1, 0.9)
    with pytest.raises(gt.THCError, match="gradient buffer's size"):
        comm.set_update(gt.GPUTensor(5), None, 0.1, 0.0)
    comm.set_update(fw, None, 0.1, 0.0)
    comm.launch(0)
    comm.wait()
    np.testing.assert_allclose(fw.float(), w0 - np.float32(0.1) * grad, rtol=1e-6, atol=1e-7)
    comm.close()

"""Stall reporting of the tensor-core kernels: a bounded wait that runs out must return control, raise the
stall flags and surface as an error at the next call that synchronises with the host -- and the library must
work normally afterwards.  The wait that runs out here is that of a one-warp probe kernel on a barrier nobody
arrives on (a few thousand SM cycles); nothing faults and nothing waits without bound."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gt():
    import mcw_cppamp_torch_b200 as m
    m.lib().THGPUInit()
    return m


def _gemm_roundtrip(gt):
    a = np.arange(300 * 40, dtype=np.float32).reshape(300, 40) / 1000
    b = np.ones((40, 70), np.float32)
    r = gt.GPUTensor(300, 70).fill(0)
    r.addmm(0.0, 1.0, gt.gpu(a), gt.gpu(b))
    return r.float(), a @ b


def test_wait_that_runs_out_becomes_an_error_at_the_next_sync(gt):
    L = gt.lib()
    L.THGPUSynchronize()
    L.THGPUStallProbe(4096)
    # the report names the wait that ran out first
    with pytest.raises(gt.THCError, match=r"pipeline stall; first report: the stall probe, code 11"):
        L.THGPUSynchronize()
    # the flags are cleared by the report: the next tensor-core product runs and is correct
    got, want = _gemm_roundtrip(gt)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)


def test_kernels_queued_behind_a_stall_leave_without_work_and_every_sync_point_reports(gt):
    L = gt.lib()
    a = gt.gpu(np.ones((300, 40), np.float32))
    b = gt.gpu(np.ones((40, 70), np.float32))
    r = gt.GPUTensor(300, 70).fill(-1)
    L.THGPUSynchronize()
    L.THGPUStallProbe(2048)
    r.addmm(0.0, 1.0, a, b)            # queued behind the stalled probe: must not write
    with pytest.raises(gt.THCError, match="pipeline stall"):
        r.float()                       # a device-to-host copy is a synchronisation point
    assert (r.float() == -1).all()      # the product did no work, and the error was reported once
    r.addmm(0.0, 1.0, a, b)
    assert (r.float() == 40).all()
    # the scalar-returning reductions report too
    L.THGPUStallProbe(2048)
    with pytest.raises(gt.THCError, match="pipeline stall"):
        r.sum()
    assert r.sum() == 300 * 70 * 40


def test_host_side_flag_alone_is_reported(gt):
    L = gt.lib()
    L.THGPUSynchronize()
    L.THGPUStallProbe(-1)               # marks the host word only, no kernel
    with pytest.raises(gt.THCError, match="pipeline stall"):
        L.THGPUSynchronize()
    L.THGPUSynchronize()


def test_wait_limit_is_a_launch_time_value(gt):
    L = gt.lib()
    old = L.THGPUGetWaitLimit()
    assert old == 1 << 27
    L.THGPUSetWaitLimit(1 << 20)
    assert L.THGPUGetWaitLimit() == 1 << 20
    got, want = _gemm_roundtrip(gt)     # a short limit does not disturb a healthy kernel
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)
    with pytest.raises(gt.THCError, match="wait limit"):
        L.THGPUSetWaitLimit(5)
    L.THGPUSetWaitLimit(old)

"""The allocation-free sum entry point (THGPUTensor_sumall_noalloc) against the regular
THGPUTensor_sumall, through the C ABI, on two calls in a row.

It exists for callers that cannot let a library allocate device memory (a region being recorded for
replay, a serving loop with a fixed memory budget, a host framework that owns every device byte).
Collected last on purpose: if it ever fails, a run that stops at the first failure has already run
everything else.  It must pass on its own in a fresh process and after the rest of the suite."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_sumall_noalloc_matches_sumall_twice_in_a_row():
    import mcw_cppamp_torch_b200 as gt
    L = gt.lib()
    L.THGPUInit()
    rs = np.random.RandomState(123)
    a = rs.standard_normal(3_000_001).astype(np.float32)          # 92 blocks, ragged tail
    b = (rs.standard_normal(70_001) * 10 + 3).astype(np.float32)   # fewer blocks than the first call
    xa, xb = gt.gpu(a), gt.gpu(b)
    out = gt.GPUTensor(2).fill(-1.0)
    stream = L.THGPUGetStream()
    base = out.data_ptr()
    # two calls back to back on the same stream, sharing the library's fixed scratch array
    assert L.THGPUTensor_sumall_noalloc(C.c_void_p(xa.data_ptr()), a.size, C.c_void_p(base), stream) == 0
    assert L.THGPUTensor_sumall_noalloc(C.c_void_p(xb.data_ptr()), b.size, C.c_void_p(base + 4), stream) == 0
    got = out.float()                                              # synchronises the stream
    want = np.array([L.THGPUTensor_sumall(xa.cdata), L.THGPUTensor_sumall(xb.cdata)], np.float32)
    assert np.all(np.abs(got - want) <= 1e-5 + 1e-4 * np.abs(want)), (got, want)
    exact = np.array([a.astype(np.float64).sum(), b.astype(np.float64).sum()])
    assert np.all(np.abs(got - exact) <= 1e-5 + 1e-4 * np.abs(exact)), (got, exact)
    # repeating the first call gives the same bits: the shared scratch carries nothing over
    assert L.THGPUTensor_sumall_noalloc(C.c_void_p(xa.data_ptr()), a.size, C.c_void_p(base + 4), stream) == 0
    again = out.float()
    assert again[1] == got[0]


def test_sumall_noalloc_rejects_sizes_beyond_its_scratch():
    import mcw_cppamp_torch_b200 as gt
    L = gt.lib()
    L.THGPUInit()
    x = gt.GPUTensor(8).fill(1.0)
    out = gt.GPUTensor(1).fill(0.0)
    for n in (0, -5, 134217728 + 1):
        with pytest.raises(gt.THCError, match="sumall_noalloc"):
            L.THGPUTensor_sumall_noalloc(C.c_void_p(x.data_ptr()), n, C.c_void_p(out.data_ptr()), L.THGPUGetStream())
    assert out.float()[0] == 0.0       # nothing was launched
    assert L.THGPUTensor_sumall_noalloc(C.c_void_p(x.data_ptr()), 8, C.c_void_p(out.data_ptr()), L.THGPUGetStream()) == 0
    assert out.float()[0] == 8.0

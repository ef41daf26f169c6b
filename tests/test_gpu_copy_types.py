"""Copies between torch.GPUTensor and the seven host tensor / storage types of TH (Byte, Char, Short, Int, Long,
Float, Double), both directions (gputorch/lib/THC/THCTensorCopy.h:8-22, THCStorageCopy.h:10-27).  The values
must equal TH's own conversions, which are C casts: `(float)x` towards the device, `(type)x` back."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

DTYPES = [np.uint8, np.int8, np.int16, np.int32, np.int64, np.float32, np.float64]


@pytest.fixture(scope="module")
def gt():
    import mcw_cppamp_torch_b200 as m
    m.lib().THGPUInit()
    return m


def _values(dtype, shape, seed):
    g = np.random.RandomState(seed)
    if np.issubdtype(dtype, np.integer):
        info = np.iinfo(dtype)
        lo, hi = max(info.min, -(1 << 22)), min(info.max, 1 << 22)     # exactly representable in float32
        return g.randint(lo, hi + 1, size=shape).astype(dtype)
    return (g.standard_normal(shape) * 1000).astype(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_host_to_device_equals_a_c_cast(gt, dtype):
    for shape in ((1,), (7,), (5, 9), (3, 4, 10), (1031,)):
        a = _values(dtype, shape, len(shape))
        x = gt.gpu(a)
        assert x.size() == shape
        got = x.float()
        assert got.dtype == np.float32 and np.array_equal(got, a.astype(np.float32)), (dtype, shape)


@pytest.mark.parametrize("dtype", DTYPES)
def test_device_to_host_truncates_like_th(gt, dtype):
    g = np.random.RandomState(3)
    f = (g.standard_normal((6, 11)) * 50).astype(np.float32)      # fractional, both signs, inside every range
    if dtype == np.uint8:
        f = np.abs(f)
    x = gt.gpu(f)
    got = x._to_host(dtype, None)
    want = f.astype(np.float64) if dtype == np.float64 else np.trunc(f).astype(dtype) if np.issubdtype(dtype, np.integer) else f
    assert got.dtype == dtype and np.array_equal(got, want)


@pytest.mark.parametrize("dtype", [np.float64, np.int16, np.uint8])
def test_strided_on_both_sides(gt, dtype):
    a = _values(dtype, (8, 12), 5)
    view = a[::2, 1::3]                                           # non-contiguous host source
    dev = gt.GPUTensor(4, 4).fill(-7)
    dev.t().copy(view)                                            # non-contiguous device destination
    assert np.array_equal(dev.float(), view.astype(np.float32).T)
    back = np.full((8, 8), 99, dtype)
    dev._to_host(dtype, back[::2, ::2])                           # non-contiguous host destination
    assert np.array_equal(back[::2, ::2], view.T.astype(np.float32).astype(dtype))
    assert (back[1::2] == 99).all() and (back[:, 1::2] == 99).all()


def test_sizes_may_differ_when_element_counts_agree_and_errors(gt):
    a = np.arange(24, dtype=np.float64)
    x = gt.GPUTensor(4, 6)
    x.copy(a)
    assert np.array_equal(x.float().ravel(), a.astype(np.float32))
    with pytest.raises(gt.THCError, match="sizes do not match"):
        x.copy(np.zeros(23, np.int32))
    with pytest.raises(gt.THCError, match="sizes do not match"):
        x.double(np.zeros((5, 5)))


@pytest.mark.parametrize("dtype", DTYPES)
def test_storage_copies(gt, dtype):
    from mcw_cppamp_torch_b200._lib import HOST_TYPES
    from mcw_cppamp_torch_b200.tensor import _TH_NAME
    L = gt.lib()
    name = _TH_NAME[np.dtype(dtype)]
    storage_t = HOST_TYPES[name][1]
    a = _values(dtype, (1000,), 11)
    if not np.issubdtype(dtype, np.integer):
        a = np.trunc(a)
    hs = storage_t()
    hs.data = C.cast(C.c_void_p(a.ctypes.data), type(hs.data)); hs.size = a.size; hs.refcount = 1
    ds = L.THGPUStorage_newWithSize(a.size)
    getattr(L, "THGPUStorage_copy" + name)(ds, C.byref(hs))
    back = np.zeros_like(a)
    hb = storage_t()
    hb.data = C.cast(C.c_void_p(back.ctypes.data), type(hb.data)); hb.size = back.size; hb.refcount = 1
    getattr(L, "TH%sStorage_copyGPU" % name)(C.byref(hb), ds)
    assert np.array_equal(back, a)
    assert L.THGPUStorage_get(ds, 17) == np.float32(a[17])
    hb.size = 5
    with pytest.raises(gt.THCError, match="size does not match"):
        getattr(L, "TH%sStorage_copyGPU" % name)(C.byref(hb), ds)
    L.THGPUStorage_free(ds)


def test_a_double_model_converts_with_gpu(gt, oracle_port):
    """Torch7's default tensor type is Double: `model:gpu()` of an unmodified model copies Double parameters
    (gputorch/Tensor.lua:7-25, mcw_nn/Module.lua:116-148)."""
    g = oracle_port.rng(4)
    m = gt.nn.SpatialConvolutionMM(3, 8, 3, 3, rng=g)
    w32 = m.weight.copy()
    m.weight, m.bias = m.weight.astype(np.float64), m.bias.astype(np.float64)
    m.gradWeight, m.gradBias = m.gradWeight.astype(np.float64), m.gradBias.astype(np.float64)
    m.gpu()
    assert np.array_equal(m.weight.float(), w32)
    x = g.uniform((2, 3, 8, 8), -1, 1)
    out = m.forward(gt.gpu(x.astype(np.float64))).double()
    want = oracle_port.conv_forward(x, w32, m.bias.float(), 3, 3, 1, 1, 0)
    np.testing.assert_allclose(out, want, rtol=1e-4, atol=1e-5)

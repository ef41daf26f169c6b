"""torch.GPUTensor copies, elementwise math and reductions on the device vs the CPU oracle.
Bit-exact for copies, add/cadd/cmul, max and indices; sums within rel 1e-4 / abs 1e-5 of TH's
double-accumulated value (they are usually bit-equal)."""
import os

import numpy as np
import pytest

from util import close

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu.npz"))


@pytest.fixture(scope="module")
def gt():
    import mcw_cppamp_torch_b200 as m
    m.lib().THGPUInit()
    return m


def test_copies_are_exact(gt, oracle_port):
    g = oracle_port.rng(1)
    a = g.normal((37, 53))
    x = gt.gpu(a)
    assert np.array_equal(x.float(), a)
    assert np.array_equal(x.clone().float(), a)
    assert np.array_equal(x.t().float(), a.T)                       # strided D2H
    assert np.array_equal(x.t().contiguous().float(), a.T)          # tiled transpose copy
    assert np.array_equal(x.narrow(2, 5, 11).float(), a[:, 4:15])   # narrowed view
    assert np.array_equal(x.select(1, 7).float(), a[6])
    y = gt.GPUTensor(53, 37)
    y.t().copy(x)                                                   # transposed destination
    assert np.array_equal(y.float(), a.T)
    z = gt.GPUTensor(53 * 37)
    z.copy(x.t())                                                   # different shapes, same count
    assert np.array_equal(z.float(), a.T.reshape(-1))
    # host -> strided device view
    w = gt.GPUTensor(53, 37).fill(0)
    w.t().copy(a)
    assert np.array_equal(w.float(), a.T)
    # non-contiguous host source
    assert np.array_equal(gt.GPUTensor(53, 37).copy(a.T).float(), a.T)
    b = g.normal((3, 4, 5, 6))
    t4 = gt.gpu(b)
    assert np.array_equal(t4.transpose(2, 4).contiguous().float(), b.transpose(0, 3, 2, 1))
    assert np.array_equal(t4.transpose(1, 3).float(), b.transpose(2, 1, 0, 3))


def test_storage_and_scalar_access(gt):
    L = gt.lib()
    x = gt.GPUTensor(5).fill(2.5)
    L.THGPUTensor_set1d(x.cdata, 3, 7.0)
    assert L.THGPUTensor_get1d(x.cdata, 3) == 7.0 and L.THGPUTensor_get1d(x.cdata, 0) == 2.5
    x.resize(3, 4)      # grows the storage, keeps the leading data
    assert x.float().reshape(-1)[:5].tolist() == [2.5, 2.5, 2.5, 7.0, 2.5]
    e = gt.GPUTensor()
    assert e.dim() == 0 and e.nElement() == 0 and e.float().size == 0
    with pytest.raises(gt.THCError):
        gt.GPUTensor(3).copy(gt.GPUTensor(4))


@pytest.mark.parametrize("shape", [(48, 80), (1, 7), (129, 33), (1000, 3)])
def test_elementwise_exact(gt, oracle_port, shape):
    g = oracle_port.rng(shape[0])
    X, Y = g.normal(shape), g.normal(shape)
    Zt = g.normal(shape[::-1])
    x, y, z = gt.gpu(X), gt.gpu(Y), gt.gpu(Zt).t()
    p = oracle_port
    R = gt.GPUTensor
    assert np.array_equal(R().add(x, 0.75).float(), p.add(X, 0.75))
    assert np.array_equal(R().add(z, 0.75).float(), p.add(Zt.T, 0.75))
    assert np.array_equal(R().add(x, -1.25, y).float(), p.cadd(X, -1.25, Y))
    assert np.array_equal(R().add(x, -1.25, z).float(), p.cadd(X, -1.25, Zt.T))
    assert np.array_equal(R().add(z, -1.25, x).float(), p.cadd(Zt.T, -1.25, X))
    assert np.array_equal(R().add(z, 3.0, z).float(), p.cadd(Zt.T, 3.0, Zt.T))
    assert np.array_equal(R().cmul(x, y).float(), p.cmul(X, Y))
    assert np.array_equal(R().cmul(z, y).float(), p.cmul(Zt.T, Y))
    # transposed destination
    d = R(*shape[::-1])
    d.t().cmul(x, z)
    assert np.array_equal(d.float(), p.cmul(X, Zt.T).T)
    # in place
    assert np.array_equal(x.clone().add(2.0).float(), p.add(X, 2.0))
    assert np.array_equal(x.clone().add(y).float(), p.cadd(X, 1.0, Y))
    assert np.array_equal(x.clone().cmul(y).float(), p.cmul(X, Y))
    assert np.array_equal(x.clone().mul(0.5).float(), X * np.float32(0.5))
    assert np.array_equal(x.clone().div(3.0).float(), X / np.float32(3.0))
    assert np.array_equal(R().cdiv(x, y).float(), X / Y)


def test_elementwise_golden(gt):
    X, Y, Zt = G["m_X"], G["m_Y"], G["m_Zt"]
    x, y, z = gt.gpu(X), gt.gpu(Y), gt.gpu(Zt).t()
    R = gt.GPUTensor
    assert np.array_equal(R().add(x, 0.75).float(), G["m_add"])
    assert np.array_equal(R().add(x, -1.25, y).float(), G["m_cadd"])
    assert np.array_equal(R().add(x, -1.25, z).float(), G["m_cadd_t"])
    assert np.array_equal(R().cmul(x, y).float(), G["m_cmul"])
    assert np.array_equal(R().cmul(z, y).float(), G["m_cmul_t"])


def test_unaligned_and_odd_sizes(gt, oracle_port):
    g = oracle_port.rng(3)
    a = g.normal((1031,))
    x = gt.gpu(a)
    v = x.narrow(1, 2, 1001)          # 4-byte-aligned only view
    assert np.array_equal(gt.GPUTensor().add(v, 1.0).float(), a[1:1002] + np.float32(1.0))
    assert abs(v.sum() - float(a[1:1002].astype(np.float64).sum())) <= 1e-5 + 1e-4 * abs(a[1:1002].sum())
    assert v.max() == a[1:1002].max() and v.min() == a[1:1002].min()


@pytest.mark.parametrize("shape", [(48, 80), (257, 1031), (5, 3), (1, 9), (2048, 130)])
def test_reductions(gt, oracle_port, shape):
    g = oracle_port.rng(7 + shape[1])
    X = g.normal(shape)
    X.reshape(-1)[::7] = 0.5                      # ties
    Zt = g.normal(shape[::-1])
    p = oracle_port
    for a, t in ((X, gt.gpu(X)), (Zt.T, gt.gpu(Zt).t())):
        close(np.float32(t.sum()), np.float32(p.sumall(a)), what="sumall")
        assert t.max() == p.maxall(a)
        assert t.min() == a.min()
        for dim in (0, 1):
            close(t.sum(dim + 1).float().reshape(-1), p.sum_dim(a, dim), what="sum(dim)")
            v, i = t.max(dim + 1)
            ov, oi = p.max_dim(a, dim)
            assert v.size() == tuple(1 if d == dim else s for d, s in enumerate(shape))
            assert np.array_equal(v.float().reshape(-1), ov)
            assert np.array_equal(i.float().reshape(-1), (oi + 1).astype(np.float32))   # 1-based, first max wins
            v, i = t.min(dim + 1)
            assert np.array_equal(v.float().reshape(-1), a.min(axis=dim))
            assert np.array_equal(i.float().reshape(-1), (a.argmin(axis=dim) + 1).astype(np.float32))
            close(t.mean(dim + 1).float().reshape(-1), a.astype(np.float64).mean(axis=dim).astype(np.float32), what="mean")
    close(np.float32(gt.gpu(X).dot(gt.gpu(X))), np.float32((X.astype(np.float64) ** 2).sum()), what="dot")


def test_reductions_golden(gt):
    X, Zt = G["m_X"], G["m_Zt"]
    x, z = gt.gpu(X), gt.gpu(Zt).t()
    close(np.array([x.sum(), z.sum()], np.float32), G["m_sumall"].astype(np.float32))
    assert x.max() == G["m_maxall"][0] and z.max() == G["m_maxall"][1]
    for dim in (0, 1):
        for t, suf in ((x, ""), (z, "_t")):
            close(t.sum(dim + 1).float().reshape(-1), G["m_sum%d%s" % (dim, suf)])
            v, i = t.max(dim + 1)
            assert np.array_equal(v.float().reshape(-1), G["m_max%d%s" % (dim, suf)])
            assert np.array_equal(i.float().reshape(-1), (G["m_argmax%d%s" % (dim, suf)] + 1).astype(np.float32))


def test_reductions_3d_and_4d(gt, oracle_port):
    g = oracle_port.rng(21)
    a = g.normal((6, 7, 33))
    t = gt.gpu(a)
    for dim in range(3):
        close(t.sum(dim + 1).float(), a.astype(np.float64).sum(axis=dim, keepdims=True).astype(np.float32), what="sum3d")
        v, i = t.max(dim + 1)
        assert np.array_equal(v.float(), a.max(axis=dim, keepdims=True))
        assert np.array_equal(i.float(), (a.argmax(axis=dim) + 1).astype(np.float32).reshape(v.size()))
    b = g.normal((3, 4, 5, 6))
    t = gt.gpu(b).transpose(2, 4)          # non-contiguous 4-D source
    bt = b.transpose(0, 3, 2, 1)
    close(t.sum(2).float(), bt.astype(np.float64).sum(axis=1, keepdims=True).astype(np.float32), what="sum4d")


def test_full_size_elementwise_and_reductions(gt, oracle_port):
    """The tensor-math configuration's 8192 x 8192 operands; checked by exact numpy equivalents
    (single fp32 operations) and order-free properties."""
    n = 8192
    rs = np.random.RandomState(5)
    X = rs.standard_normal((n, n)).astype(np.float32)
    Y = rs.standard_normal((n, n)).astype(np.float32)
    x, y = gt.gpu(X), gt.gpu(Y)
    r = gt.GPUTensor()
    assert np.array_equal(r.add(x, 0.5, y).float(), X + np.float32(0.5) * Y)
    assert np.array_equal(r.cmul(x, y.t()).float(), X * Y.T)
    assert np.array_equal(r.add(x.t(), 1.0).float(), X.T + np.float32(1.0))
    s64 = X.astype(np.float64).sum()
    assert abs(x.sum() - s64) <= 1e-5 + 1e-4 * abs(s64)
    assert abs(x.t().sum() - s64) <= 1e-5 + 1e-4 * abs(s64)
    assert x.max() == X.max() and x.t().max() == X.max()
    for t, a in ((x, X), (x.t(), X.T)):
        for dim in (0, 1):
            close(t.sum(dim + 1).float().reshape(-1), a.astype(np.float64).sum(axis=dim).astype(np.float32), what="sum")
            v, i = t.max(dim + 1)
            assert np.array_equal(v.float().reshape(-1), a.max(axis=dim))
            assert np.array_equal(i.float().reshape(-1), (a.argmax(axis=dim) + 1).astype(np.float32))

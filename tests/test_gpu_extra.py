"""The rest of the tensor-math surface (zeros / ones / reshape, prodall / prod, renorm, indexSelect / indexCopy /
indexFill) and the SoftMax and SpatialAveragePooling operators on the device, against the CPU oracle and the
golden vectors made from the reference's own TH / nn build."""
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


def test_zeros_ones_reshape(gt):
    z = gt.GPUTensor().zeros(3, 5)
    o = gt.GPUTensor(2).ones(4, 2, 3)
    assert z.size() == (3, 5) and not z.float().any()
    assert o.size() == (4, 2, 3) and (o.float() == 1).all()
    a = np.arange(24, dtype=np.float32).reshape(4, 6)
    r = gt.GPUTensor().reshape(gt.gpu(a).t(), 3, 8)              # logical order of the transposed view
    assert np.array_equal(r.float(), a.T.reshape(3, 8))
    x = gt.gpu(a)
    x.reshape(x, 2, 12)                                          # in place
    assert np.array_equal(x.float(), a.reshape(2, 12))
    with pytest.raises(gt.THCError, match="sizes do not match"):
        gt.GPUTensor().reshape(gt.gpu(a), 5, 5)


def test_products_golden_and_views(gt, oracle_port):
    T = G["x_T"]
    x = gt.gpu(T)
    assert abs(x.prod() - G["x_prodall"][0]) <= 1e-4 * abs(G["x_prodall"][0])
    for dim in (0, 1, 2):
        close(x.prod(dim + 1).float(), G["x_prod%d" % dim], what="prod dim %d" % dim)
    g = oracle_port.rng(3)
    big = g.uniform((300, 257), 0.99, 1.01)
    xb = gt.gpu(big)
    close(xb.prod(1).float(), oracle_port.prod_dim(big, 0)); close(xb.prod(2).float(), oracle_port.prod_dim(big, 1))
    close(xb.t().prod(1).float(), oracle_port.prod_dim(big.T, 0))           # non-contiguous source
    want = float(np.float32(oracle_port.prodall(big)))                       # the C API returns a float
    assert want != 0 and abs(xb.prod() - want) <= 1e-4 * abs(want)
    xb.prod(xb, 2)                                                          # result into the source itself
    close(xb.float(), oracle_port.prod_dim(big, 1))


def test_renorm_golden_and_rows_below_the_limit_untouched(gt, oracle_port):
    T = G["x_T"]
    for dim in (0, 1, 2):
        for k, (v, m) in enumerate(((1.0, 20.0), (2.0, 5.0), (3.0, 4.5))):
            got = gt.gpu(T).renorm(v, dim + 1, m).float()
            close(got, G["x_renorm%d" % dim][k], what="renorm dim %d p %g" % (dim, v))
    g = oracle_port.rng(8)
    W = g.normal((50, 300))
    W[::2] *= 0.01                                                           # every other row stays below maxnorm
    r = gt.GPUTensor().renorm(gt.gpu(W), 2, 1, 3.0).float()
    close(r, oracle_port.renorm(W, 2.0, 0, 3.0))
    assert np.array_equal(r[::2], W[::2])
    with pytest.raises(gt.THCError, match="at least 2 dimensions"):
        gt.gpu(np.ones(5, np.float32)).renorm(2, 1, 1.0)


def test_index_operations(gt, oracle_port):
    T, idx, src = G["x_T"], G["x_idx"], G["x_src"]
    assert np.array_equal(gt.gpu(T).index(2, idx).float(), G["x_select1"])
    assert np.array_equal(gt.gpu(T).indexFill(3, idx[:2], -2.5).float(), G["x_fill2"])
    # indexCopy with a repeated position is order dependent: use distinct positions for the exact comparison
    uniq = np.array([3, 1, 6, 2], np.int64)
    assert np.array_equal(gt.gpu(T).indexCopy(2, uniq, gt.gpu(src)).float(), oracle_port.index_copy(T, 1, uniq, src))
    g = oracle_port.rng(14)
    big = g.normal((37, 129, 9))
    pick = np.array([129, 1, 64, 64, 7, 100, 2], np.int64)
    xb = gt.gpu(big)
    assert np.array_equal(xb.index(2, pick).float(), oracle_port.index_select(big, 1, pick))
    assert np.array_equal(xb.index(1, [7, 37, 2]).float(), oracle_port.index_select(big, 0, [7, 37, 2]))
    assert np.array_equal(xb.index(3, [9, 1]).float(), oracle_port.index_select(big, 2, [9, 1]))
    tv = gt.gpu(np.ascontiguousarray(big.transpose(1, 0, 2))).transpose(1, 2)     # a view shaped like `big`
    assert np.array_equal(tv.index(2, pick).float(), oracle_port.index_select(big, 1, pick))
    tv.indexFill(2, [5, 6], 3.0)                                                  # non-contiguous destination
    assert np.array_equal(tv.float(), oracle_port.index_fill(big, 1, [5, 6], 3.0))
    for bad in ([0], [130]):
        with pytest.raises(gt.THCError, match="index out of range"):
            xb.index(2, bad)
    with pytest.raises(gt.THCError, match="not equal to length of indices"):
        xb.indexCopy(2, [1, 2], gt.gpu(big))


def test_softmax_golden_and_large(gt, oracle_port):
    m = gt.nn.SoftMax()
    out = m.forward(gt.gpu(G["sm_z"])).float()
    close(out, G["sm_out"], rtol=1e-6, atol=1e-7, what="SoftMax output")
    close(m.backward(gt.gpu(G["sm_z"]), gt.gpu(G["sm_go"])).float(), G["sm_gi"], rtol=1e-5, atol=1e-7, what="SoftMax gradInput")
    g = oracle_port.rng(6)
    z = g.normal((128, 1000), 0, 4)
    out = m.forward(gt.gpu(z)).float()
    want = oracle_port.softmax_forward(z)
    close(out, want, rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(out.sum(axis=1), 1.0, rtol=1e-5)
    go = g.normal(z.shape)
    close(m.backward(gt.gpu(z), gt.gpu(go)).float(), oracle_port.softmax_backward(go, want), rtol=1e-4, atol=1e-6)
    v = g.normal((17,))
    close(m.forward(gt.gpu(v)).float(), oracle_port.softmax_forward(v), rtol=1e-6, atol=1e-7)   # 1-D input


def test_average_pooling_is_bit_exact(gt, oracle_port):
    x = G["ap_x"]
    for name in ("ap22", "ap32", "ap_odd"):
        kH, kW, dH, dW = (int(v) for v in G[name + "_cfg"])
        m = gt.nn.SpatialAveragePooling(kW, kH, dW, dH)
        assert np.array_equal(m.forward(gt.gpu(x)).float(), G[name + "_out"])
        assert np.array_equal(m.backward(gt.gpu(x), gt.gpu(G[name + "_go"])).float(), G[name + "_gi"])
    g = oracle_port.rng(10)
    big = g.normal((8, 64, 55, 55))
    for kH, kW, dH, dW in ((3, 3, 2, 2), (2, 2, 2, 2), (5, 3, 1, 4)):
        m = gt.nn.SpatialAveragePooling(kW, kH, dW, dH)
        out = m.forward(gt.gpu(big)).float()
        assert np.array_equal(out, oracle_port.sumpool_forward(big, kH, kW, dH, dW))
        go = g.normal(out.shape)
        assert np.array_equal(m.backward(gt.gpu(big), gt.gpu(go)).float(),
                              oracle_port.sumpool_backward(go, big.shape, kH, kW, dH, dW))
    m = gt.nn.SpatialAveragePooling(2, 2, 2, 2)
    assert m.forward(gt.gpu(big[0])).size() == (64, 27, 27)                 # 3-D input
    with pytest.raises(gt.THCError, match="smaller than kernel"):
        gt.nn.SpatialAveragePooling(9, 9).forward(gt.GPUTensor(1, 4, 4))

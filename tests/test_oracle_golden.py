"""The CPU restatement against golden vectors produced by the reference's own CPU code
(tests/golden/make_golden.py).  Runs anywhere: needs neither the reference tree nor a GPU."""
import os

import numpy as np
import pytest

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu.npz"))


def test_rng_known_answers(oracle_port):
    g = oracle_port.rng(int(G["rng_seed"][0]))
    assert np.array_equal(g.uniform((64,), -1, 1), G["rng_uniform_m1_1"])
    assert np.array_equal(g.normal((65,)), G["rng_normal_0_1"])
    assert np.array_equal(g.uniform((8,), 0, 1), G["rng_uniform_after"])


def test_conv_block_stride1_bit_exact(oracle_port):
    N, C, H, W, K, k, d, pad = G["s1_cfg"]
    x, w, b = G["s1_x"], G["s1_w"], G["s1_b"]
    conv = oracle_port.conv_forward(x, w, b, k, k, d, d, pad)
    assert np.array_equal(conv, G["s1_conv"])
    relu = oracle_port.threshold_forward(conv)
    assert np.array_equal(relu, G["s1_relu"])
    pool, ind = oracle_port.maxpool_forward(relu, 3, 3, 2, 2)
    assert np.array_equal(pool, G["s1_pool"]) and np.array_equal(ind, G["s1_ind"])
    g_relu = oracle_port.maxpool_backward(G["s1_go"], ind, relu.shape, 2, 2)
    assert np.array_equal(g_relu, G["s1_g_relu"])
    g_conv = oracle_port.threshold_backward(conv, g_relu)
    assert np.array_equal(g_conv, G["s1_g_conv"])
    assert np.array_equal(oracle_port.conv_grad_input(g_conv, w, x.shape, k, k, d, d, pad), G["s1_gi"])
    gw, gb = np.zeros_like(w), np.zeros_like(b)
    oracle_port.conv_acc_grad(x, g_conv, gw, gb, 1.0, k, k, d, d, pad)
    assert np.array_equal(gw, G["s1_gw"]) and np.array_equal(gb, G["s1_gb"])


def test_conv_stride4_within_tolerance(oracle_port):
    N, C, H, W, K, k, d, pad = G["s4_cfg"]
    x, w, b, go = G["s4_x"], G["s4_w"], G["s4_b"], G["s4_go"]
    tol = dict(rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(oracle_port.conv_forward(x, w, b, k, k, d, d, pad), G["s4_conv"], **tol)
    np.testing.assert_allclose(oracle_port.conv_grad_input(go, w, x.shape, k, k, d, d, pad), G["s4_gi"], **tol)
    gw, gb = np.zeros_like(w), np.zeros_like(b)
    oracle_port.conv_acc_grad(x, go, gw, gb, 1.0, k, k, d, d, pad)
    np.testing.assert_allclose(gw, G["s4_gw"], **tol)
    np.testing.assert_allclose(gb, G["s4_gb"], **tol)


@pytest.mark.parametrize("name,k,d", [("p32", 3, 2), ("p22", 2, 2)])
def test_pool_bit_exact(oracle_port, name, k, d):
    x = G[name + "_x"]
    o, i = oracle_port.maxpool_forward(x, k, k, d, d)
    assert np.array_equal(o, G[name + "_out"]) and np.array_equal(i, G[name + "_ind"])
    assert np.array_equal(oracle_port.maxpool_backward(G[name + "_go"], i, x.shape, d, d), G[name + "_gi"])


def test_tensor_math_bit_exact(oracle_port):
    X, Y, Zt = G["m_X"], G["m_Y"], G["m_Zt"]
    p = oracle_port
    assert np.array_equal(p.add(X, 0.75), G["m_add"])
    assert np.array_equal(p.cadd(X, -1.25, Y), G["m_cadd"])
    assert np.array_equal(p.cadd(X, -1.25, Zt.T), G["m_cadd_t"])
    assert np.array_equal(p.cmul(X, Y), G["m_cmul"])
    assert np.array_equal(p.cmul(Zt.T, Y), G["m_cmul_t"])
    assert np.array_equal(np.array([p.sumall(X), p.sumall(Zt.T)]), G["m_sumall"])
    assert np.array_equal(np.array([p.maxall(X), p.maxall(Zt.T)], np.float32), G["m_maxall"])
    for dim in (0, 1):
        assert np.array_equal(p.sum_dim(X, dim), G["m_sum%d" % dim])
        assert np.array_equal(p.sum_dim(Zt.T, dim), G["m_sum%d_t" % dim])
        for src, suf in ((X, ""), (Zt.T, "_t")):
            v, i = p.max_dim(src, dim)
            assert np.array_equal(v, G["m_max%d%s" % (dim, suf)])
            assert np.array_equal(i, G["m_argmax%d%s" % (dim, suf)])
    A, B, Cm, Bt = G["m_A"], G["m_B"], G["m_C"], G["m_Bt"]
    assert np.array_equal(p.addmm(1.0, Cm, 1.0, A, B), G["m_addmm"])
    assert np.array_equal(p.addmm(0.5, Cm, 2.0, A, B), G["m_addmm_b"])
    assert np.array_equal(p.addmm(0.5, Cm, 2.0, A, Bt.T), G["m_addmm_t"])


def test_logsoftmax_bit_exact(oracle_port):
    out = oracle_port.logsoftmax_forward(G["l_z"])
    assert np.array_equal(out, G["l_out"])
    assert np.array_equal(oracle_port.logsoftmax_backward(G["l_go"], out), G["l_gi"])


def test_pointwise_and_norms_bit_exact(oracle_port):
    from util import pointwise_cases
    X, Y = G["m_X"], G["m_Y"]
    p = oracle_port
    for key, name, a, b, c, v1, v2 in pointwise_cases(X, Y):
        assert np.array_equal(p.pointwise(name, a, b, c, v1, v2), G["pw_" + key]), key
    assert np.array_equal(np.array([p.normall(X, v) for v in (0.0, 1.0, 2.0, 3.5)]), G["pw_normall"])
    assert np.array_equal(np.array([p.dist(X, Y, v) for v in (1.0, 2.0, 2.5)]), G["pw_dist"])
    assert np.array_equal(np.array([p.varall(X)]), G["pw_varall"])
    for dim in (0, 1):
        assert np.array_equal(np.stack([p.norm_dim(X, v, dim) for v in (0.0, 1.0, 2.0, 3.0)]), G["pw_norm%d" % dim])


EXTRA_RENORM = ((1.0, 20.0), (2.0, 5.0), (3.0, 4.5))
AVG_POOLS = ("ap22", "ap32", "ap_odd")


def test_prod_renorm_index_softmax_average_pooling_bit_exact(oracle_port):
    p = oracle_port
    T, idx, src = G["x_T"], G["x_idx"], G["x_src"]
    assert p.prodall(T) == G["x_prodall"][0]
    for dim in (0, 1, 2):
        assert np.array_equal(p.prod_dim(T, dim), G["x_prod%d" % dim])
        assert np.array_equal(np.stack([p.renorm(T, v, dim, m) for v, m in EXTRA_RENORM]), G["x_renorm%d" % dim])
    assert np.array_equal(p.index_select(T, 1, idx), G["x_select1"])
    assert np.array_equal(p.index_copy(T, 1, idx, src), G["x_copy1"])
    assert np.array_equal(p.index_fill(T, 2, idx[:2], -2.5), G["x_fill2"])
    out = p.softmax_forward(G["sm_z"])
    assert np.array_equal(out, G["sm_out"])
    assert np.array_equal(p.softmax_backward(G["sm_go"], out), G["sm_gi"])
    for name in AVG_POOLS:
        kH, kW, dH, dW = (int(v) for v in G[name + "_cfg"])
        assert np.array_equal(p.sumpool_forward(G["ap_x"], kH, kW, dH, dW), G[name + "_out"])
        assert np.array_equal(p.sumpool_backward(G[name + "_go"], G["ap_x"].shape, kH, kW, dH, dW), G[name + "_gi"])


def test_package_generator_follows_the_th_stream(oracle_port):
    """mcw_cppamp_torch_b200.random.THGenerator (what the benchmark and the examples draw from) against the pinned
    restatement of THRandom.c and the reference's own numbers."""
    from mcw_cppamp_torch_b200.random import THGenerator
    t = THGenerator(int(G["rng_seed"][0]))
    assert np.array_equal(t.uniform((64,), -1, 1), G["rng_uniform_m1_1"])
    assert np.array_equal(t.normal((65,)), G["rng_normal_0_1"])            # an odd count leaves a cached value
    assert np.array_equal(t.uniform((8,), 0, 1), G["rng_uniform_after"])
    g, t = oracle_port.rng(77), THGenerator(77)
    for shape, kind in (((3, 5), "n"), ((7,), "u"), ((1,), "n"), ((4, 4), "n"), ((9,), "u"), ((10001,), "n")):
        if kind == "n":
            assert np.array_equal(g.normal(shape, 0.5, 2.0), t.normal(shape, 0.5, 2.0))
        else:
            assert np.array_equal(g.uniform(shape, -3, 4), t.uniform(shape, -3, 4))
    lab = THGenerator(5).labels(1000, 1000)
    assert lab.min() >= 1 and lab.max() <= 1000 and lab.dtype == np.float32

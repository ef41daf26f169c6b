"""The CPU restatement (oracle/oracle.c) against the reference's own compiled CPU code
(oracle/_ref/liboracle_ref.so: TH + mcw_nn generic kernels, unmodified).  Bit-exact wherever the
reference can run the case (its MM conv rejects stride > 1); tolerance only on the stride route,
where the reference uses a different algorithm (conv2Dmm) and hence another summation order."""
import numpy as np
import pytest


def test_rng_stream_matches_th(oracle_port, oracle_ref):
    for seed in (1, 1234, 2**31 + 7):
        a, b = oracle_port.rng(seed), oracle_ref.rng(seed)
        assert np.array_equal(a.uniform((1000,), -1, 1), b.uniform((1000,), -1, 1))
        # odd count leaves a cached Box-Muller value behind; the next call must consume it
        assert np.array_equal(a.normal((7,)), b.normal((7,)))
        assert np.array_equal(a.normal((2000,), 0.5, 2.0), b.normal((2000,), 0.5, 2.0))
        assert np.array_equal(a.uniform((3, 5), 0, 1000), b.uniform((3, 5), 0, 1000))


@pytest.mark.parametrize("N,C,H,W,K,k,pad", [
    (2, 3, 12, 11, 8, 3, 0), (3, 5, 9, 9, 16, 5, 2), (1, 4, 7, 8, 8, 3, 1), (2, 1, 6, 6, 3, 1, 0),
    (2, 16, 13, 13, 24, 3, 1),
])
def test_conv_stride1_bit_exact(oracle_port, oracle_ref, N, C, H, W, K, k, pad):
    g = oracle_port.rng(42 + N + C)
    x = g.uniform((N, C, H, W), -1, 1)
    s = 1.0 / np.sqrt(C * k * k)
    w = g.uniform((K, C * k * k), -s, s)
    b = g.uniform((K,), -s, s)
    out_p = oracle_port.conv_forward(x, w, b, k, k, 1, 1, pad)
    out_r = oracle_ref.conv_forward(x, w, b, k, k, 1, 1, pad)
    assert out_p.shape == out_r.shape
    assert np.array_equal(out_p, out_r)
    go = g.normal(out_p.shape)
    gw0 = g.normal(w.shape)  # non-zero start: accGradParameters accumulates
    gb0 = g.normal(b.shape)
    gi_r, gw_r, gb_r = oracle_ref.conv_backward(x, w, go, gw0, gb0, 0.5, k, k, 1, 1, pad)
    gi_p = oracle_port.conv_grad_input(go, w, x.shape, k, k, 1, 1, pad)
    gw_p, gb_p = gw0.copy(), gb0.copy()
    oracle_port.conv_acc_grad(x, go, gw_p, gb_p, 0.5, k, k, 1, 1, pad)
    assert np.array_equal(gi_p, gi_r)
    assert np.array_equal(gw_p, gw_r)
    assert np.array_equal(gb_p, gb_r)


def test_reference_mm_conv_rejects_stride(oracle_ref):
    x = np.zeros((1, 1, 8, 8), np.float32)
    with pytest.raises(RuntimeError, match="dW must == 1"):
        oracle_ref.conv_forward(x, np.zeros((2, 9), np.float32), np.zeros(2, np.float32), 3, 3, 1, 2, 0)


@pytest.mark.parametrize("N,C,H,W,K,k,d,pad", [
    (2, 3, 23, 23, 8, 11, 4, 2), (2, 4, 12, 15, 6, 3, 2, 1), (1, 2, 9, 9, 4, 5, 3, 0), (2, 3, 10, 10, 5, 3, 1, 1),
])
def test_conv_strided_against_conv2dmm_route(oracle_port, oracle_ref, N, C, H, W, K, k, d, pad):
    g = oracle_port.rng(7)
    x = g.uniform((N, C, H, W), -1, 1)
    s = 1.0 / np.sqrt(C * k * k)
    w = g.uniform((K, C * k * k), -s, s)
    b = g.uniform((K,), -s, s)
    out_p = oracle_port.conv_forward(x, w, b, k, k, d, d, pad)
    go = g.normal(out_p.shape)
    gw0, gb0 = np.zeros_like(w), np.zeros_like(b)
    out_r, gi_r, gw_r, gb_r = oracle_ref.conv_strided(
        x, w.reshape(K, C, k, k), b, go, gw0.reshape(K, C, k, k), gb0, 1.0, d, d, pad)
    gi_p = oracle_port.conv_grad_input(go, w, x.shape, k, k, d, d, pad)
    gw_p, gb_p = gw0.copy(), gb0.copy()
    oracle_port.conv_acc_grad(x, go, gw_p, gb_p, 1.0, k, k, d, d, pad)
    tol = dict(rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(out_p, out_r, **tol)
    np.testing.assert_allclose(gi_p, gi_r, **tol)
    np.testing.assert_allclose(gw_p, gw_r.reshape(K, -1), rtol=1e-4, atol=2e-5)
    np.testing.assert_allclose(gb_p, gb_r, rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("shape,k,d", [((2, 3, 9, 11), (3, 3), (2, 2)), ((4, 7, 7), (2, 2), (2, 2)),
                                        ((1, 2, 13, 13), (3, 2), (1, 3)), ((2, 2, 6, 6), (6, 6), (1, 1))])
def test_maxpool_bit_exact(oracle_port, oracle_ref, shape, k, d):
    g = oracle_port.rng(3)
    x = g.normal(shape)
    x.reshape(-1)[::5] = 0.25  # ties: first maximum must win
    o_p, i_p = oracle_port.maxpool_forward(x, k[0], k[1], d[0], d[1])
    o_r, i_r = oracle_ref.maxpool_forward(x, k[0], k[1], d[0], d[1])
    assert np.array_equal(o_p, o_r) and np.array_equal(i_p.reshape(-1), i_r.reshape(-1))
    go = g.normal(o_p.shape)
    gi_p = oracle_port.maxpool_backward(go, i_p, x.shape, d[0], d[1])
    gi_r = oracle_ref.maxpool_backward(x, go, i_r, d[0], d[1])
    assert np.array_equal(gi_p, gi_r)


def test_threshold_bit_exact(oracle_port, oracle_ref):
    g = oracle_port.rng(5)
    x, go = g.normal((3, 4, 5, 6)), g.normal((3, 4, 5, 6))
    for th, val in ((0.0, 0.0), (0.3, -1.5)):
        assert np.array_equal(oracle_port.threshold_forward(x, th, val), oracle_ref.threshold_forward(x, th, val))
        assert np.array_equal(oracle_port.threshold_backward(x, go, th), oracle_ref.threshold_backward(x, go, th))


def test_tensor_math_bit_exact(oracle_port, oracle_ref):
    g = oracle_port.rng(11)
    X, Y = g.normal((37, 53)), g.normal((37, 53))
    Xt, Yt = g.normal((53, 37)).T, g.normal((53, 37)).T  # transposed views of shape (37, 53)
    for a, b in ((X, Y), (Xt, Y), (X, Yt), (Xt, Yt)):
        assert np.array_equal(oracle_port.add(a, 1.5), oracle_ref.add(a, 1.5))
        assert np.array_equal(oracle_port.cadd(a, -0.7, b), oracle_ref.cadd(a, -0.7, b))
        assert np.array_equal(oracle_port.cmul(a, b), oracle_ref.cmul(a, b))
        assert oracle_port.sumall(a) == oracle_ref.sumall(a)
        assert oracle_port.maxall(a) == oracle_ref.maxall(a)
        for dim in (0, 1):
            assert np.array_equal(oracle_port.sum_dim(a, dim), oracle_ref.sum_dim(a, dim))
            vp, ip = oracle_port.max_dim(a, dim)
            vr, ir = oracle_ref.max_dim(a, dim)
            assert np.array_equal(vp, vr) and np.array_equal(ip, ir)


def test_addmm_bit_exact(oracle_port, oracle_ref):
    g = oracle_port.rng(13)
    M, N, K = 19, 23, 31
    t = g.normal((M, N))
    A, B = g.normal((M, K)), g.normal((K, N))
    At, Bt = g.normal((K, M)).T, g.normal((N, K)).T
    for a in (A, At):
        for b in (B, Bt):
            for beta, alpha in ((1.0, 1.0), (0.5, 2.0), (0.0, 1.0)):
                assert np.array_equal(oracle_port.addmm(beta, t, alpha, a, b), oracle_ref.addmm(beta, t, alpha, a, b))


def test_logsoftmax_bit_exact(oracle_port, oracle_ref):
    g = oracle_port.rng(17)
    x = g.normal((6, 50), 0, 3)
    o_p, o_r = oracle_port.logsoftmax_forward(x), oracle_ref.logsoftmax_forward(x)
    assert np.array_equal(o_p, o_r)
    go = g.normal((6, 50))
    assert np.array_equal(oracle_port.logsoftmax_backward(go, o_p), oracle_ref.logsoftmax_backward(go, o_r))


def test_pointwise_and_norms_bit_exact(oracle_port, oracle_ref):
    from util import pointwise_cases
    g = oracle_port.rng(21)
    X, Y = g.normal((19, 45)), g.normal((19, 45))
    for key, name, a, b, c, v1, v2 in pointwise_cases(X, Y):
        assert np.array_equal(oracle_port.pointwise(name, a, b, c, v1, v2), oracle_ref.pointwise(name, a, b, c, v1, v2)), key
    for value in (0.0, 1.0, 2.0, 3.5):
        assert oracle_port.normall(X, value) == oracle_ref.normall(X, value)
    for value in (1.0, 2.0, 2.5):
        assert oracle_port.dist(X, Y, value) == oracle_ref.dist(X, Y, value)
    assert oracle_port.varall(X) == oracle_ref.varall(X)
    for value in (0.0, 1.0, 2.0, 3.0):
        for dim in (0, 1):
            assert np.array_equal(oracle_port.norm_dim(X, value, dim), oracle_ref.norm_dim(X, value, dim))



def _extra_cases(g):
    """(3-D tensor, index vector) shared by the pins of prod / renorm / index* below."""
    T = g.uniform((4, 6, 5), 0.5, 1.5)
    idx = np.array([3, 1, 6, 3], np.int64)         # 1-based, with a repeat
    return T, idx


def test_prod_renorm_and_index_ops_bit_exact(oracle_port, oracle_ref):
    g = oracle_port.rng(29)
    T, idx = _extra_cases(g)
    assert oracle_port.prodall(T) == oracle_ref.prodall(T)
    for dim in (0, 1, 2):
        assert np.array_equal(oracle_port.prod_dim(T, dim), oracle_ref.prod_dim(T, dim))
        for value, maxnorm in ((1.0, 20.0), (2.0, 5.0), (3.0, 4.5), (2.0, 1e9)):
            assert np.array_equal(oracle_port.renorm(T, value, dim, maxnorm), oracle_ref.renorm(T, value, dim, maxnorm))
    assert np.array_equal(oracle_port.index_select(T, 1, idx), oracle_ref.index_select(T, 1, idx))
    assert np.array_equal(oracle_port.index_select(T, 0, idx[:2]), oracle_ref.index_select(T, 0, idx[:2]))
    src = g.normal((4, 4, 5))
    assert np.array_equal(oracle_port.index_copy(T, 1, idx, src), oracle_ref.index_copy(T, 1, idx, src))
    assert np.array_equal(oracle_port.index_fill(T, 2, idx[:2], -2.5), oracle_ref.index_fill(T, 2, idx[:2], -2.5))


def test_softmax_and_average_pooling_bit_exact(oracle_port, oracle_ref):
    g = oracle_port.rng(37)
    x = g.normal((7, 33), 0, 3)
    o_p, o_r = oracle_port.softmax_forward(x), oracle_ref.softmax_forward(x)
    assert np.array_equal(o_p, o_r)
    go = g.normal((7, 33))
    assert np.array_equal(oracle_port.softmax_backward(go, o_p), oracle_ref.softmax_backward(go, o_r))
    img = g.normal((2, 3, 11, 13))
    for kH, kW, dH, dW in ((2, 2, 2, 2), (3, 3, 2, 2), (3, 2, 1, 1), (4, 5, 3, 2)):
        o_p, o_r = oracle_port.sumpool_forward(img, kH, kW, dH, dW), oracle_ref.sumpool_forward(img, kH, kW, dH, dW)
        assert np.array_equal(o_p, o_r)
        go = g.normal(o_p.shape)
        assert np.array_equal(oracle_port.sumpool_backward(go, img.shape, kH, kW, dH, dW),
                              oracle_ref.sumpool_backward(img, go, kH, kW, dH, dW))

"""Generates tests/golden/reference_cpu.npz from the reference's own compiled CPU code.

Run where the reference tree is mounted (the Makefile in oracle/ compiles it into
oracle/_ref/liboracle_ref.so):   python tests/golden/make_golden.py
Every array is produced by the reference's unmodified TH / nn code on inputs drawn from TH's own
MT19937 stream (seeds recorded in the file), so the vectors pin both the CPU restatement and the
CUDA path on machines where the reference tree does not exist."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import oracle  # noqa: E402


def main():
    oracle.build()
    ref = oracle.ref
    out = {}
    # RNG known answers
    g = ref.rng(1234)
    out["rng_seed"] = np.array([1234])
    out["rng_uniform_m1_1"] = g.uniform((64,), -1, 1)
    out["rng_normal_0_1"] = g.normal((65,))
    out["rng_uniform_after"] = g.uniform((8,), 0, 1)

    # conv block in the shape family of the single-conv-block config, stride 1 (MM route, bit-exact pin)
    g = ref.rng(2024)
    N, C, H, W, K, k, pad = 2, 3, 20, 20, 8, 5, 2
    s = 1.0 / np.sqrt(C * k * k)
    x = g.uniform((N, C, H, W), -1, 1)
    w = g.uniform((K, C * k * k), -s, s)
    b = g.uniform((K,), -s, s)
    conv = ref.conv_forward(x, w, b, k, k, 1, 1, pad)
    relu = ref.threshold_forward(conv, 0, 0)
    pool, ind = ref.maxpool_forward(relu, 3, 3, 2, 2)
    go = g.normal(pool.shape)
    g_relu = ref.maxpool_backward(relu, go, ind, 2, 2)
    g_conv = ref.threshold_backward(conv, g_relu, 0)
    gi, gw, gb = ref.conv_backward(x, w, g_conv, np.zeros_like(w), np.zeros_like(b), 1.0, k, k, 1, 1, pad)
    out.update(s1_x=x, s1_w=w, s1_b=b, s1_conv=conv, s1_relu=relu, s1_pool=pool, s1_ind=ind, s1_go=go,
               s1_g_relu=g_relu, s1_g_conv=g_conv, s1_gi=gi, s1_gw=gw, s1_gb=gb,
               s1_cfg=np.array([N, C, H, W, K, k, 1, pad]))

    # the stride-4 / pad-2 / 11x11 first layer, small spatial size (conv2Dmm route: tolerance pin)
    g = ref.rng(77)
    N, C, H, W, K, k, d, pad = 2, 3, 39, 39, 8, 11, 4, 2
    s = 1.0 / np.sqrt(C * k * k)
    x = g.uniform((N, C, H, W), -1, 1)
    w = g.uniform((K, C * k * k), -s, s)
    b = g.uniform((K,), -s, s)
    oH = (H + 2 * pad - k) // d + 1
    go = g.normal((N, K, oH, oH))
    conv, gi, gw, gb = ref.conv_strided(x, w.reshape(K, C, k, k), b, go, np.zeros((K, C, k, k), np.float32),
                                        np.zeros(K, np.float32), 1.0, d, d, pad)
    out.update(s4_x=x, s4_w=w, s4_b=b, s4_go=go, s4_conv=conv, s4_gi=gi, s4_gw=gw.reshape(K, -1), s4_gb=gb,
               s4_cfg=np.array([N, C, H, W, K, k, d, pad]))

    # overlapping and non-overlapping pooling with ties
    g = ref.rng(5)
    x = g.normal((2, 3, 13, 13))
    x.reshape(-1)[::4] = 0.5
    for name, (kk, dd) in dict(p32=(3, 2), p22=(2, 2)).items():
        o, i = ref.maxpool_forward(x, kk, kk, dd, dd)
        go = g.normal(o.shape)
        out[name + "_x"] = x
        out[name + "_out"], out[name + "_ind"], out[name + "_go"] = o, i, go
        out[name + "_gi"] = ref.maxpool_backward(x, go, i, dd, dd)

    # tensor math incl. transposed views
    g = ref.rng(99)
    X, Y = g.normal((48, 80)), g.normal((48, 80))
    Zt = g.normal((80, 48))  # used as Zt.T
    A, B, Cm = g.normal((33, 47)), g.normal((47, 29)), g.normal((33, 29))
    Bt = g.normal((29, 47))
    out.update(m_X=X, m_Y=Y, m_Zt=Zt, m_A=A, m_B=B, m_C=Cm, m_Bt=Bt)
    from util import pointwise_cases
    for key, name, a, b, c, v1, v2 in pointwise_cases(X, Y):
        out["pw_" + key] = ref.pointwise(name, a, b, c, v1, v2)
    out["pw_normall"] = np.array([ref.normall(X, v) for v in (0.0, 1.0, 2.0, 3.5)])
    out["pw_dist"] = np.array([ref.dist(X, Y, v) for v in (1.0, 2.0, 2.5)])
    out["pw_varall"] = np.array([ref.varall(X)])
    for dim in (0, 1):
        out["pw_norm%d" % dim] = np.stack([ref.norm_dim(X, v, dim) for v in (0.0, 1.0, 2.0, 3.0)])
    out["m_add"] = ref.add(X, 0.75)
    out["m_cadd"] = ref.cadd(X, -1.25, Y)
    out["m_cadd_t"] = ref.cadd(X, -1.25, Zt.T)
    out["m_cmul"] = ref.cmul(X, Y)
    out["m_cmul_t"] = ref.cmul(Zt.T, Y)
    out["m_sumall"] = np.array([ref.sumall(X), ref.sumall(Zt.T)])
    out["m_maxall"] = np.array([ref.maxall(X), ref.maxall(Zt.T)], np.float32)
    for dim in (0, 1):
        out["m_sum%d" % dim] = ref.sum_dim(X, dim)
        out["m_sum%d_t" % dim] = ref.sum_dim(Zt.T, dim)
        v, i = ref.max_dim(X, dim)
        out["m_max%d" % dim], out["m_argmax%d" % dim] = v, i
        v, i = ref.max_dim(Zt.T, dim)
        out["m_max%d_t" % dim], out["m_argmax%d_t" % dim] = v, i
    out["m_addmm"] = ref.addmm(1.0, Cm, 1.0, A, B)
    out["m_addmm_b"] = ref.addmm(0.5, Cm, 2.0, A, B)
    out["m_addmm_t"] = ref.addmm(0.5, Cm, 2.0, A, Bt.T)

    # classifier tail
    g = ref.rng(31)
    z = g.normal((5, 40), 0, 2)
    lsm = ref.logsoftmax_forward(z)
    go = g.normal((5, 40))
    out.update(l_z=z, l_out=lsm, l_go=go, l_gi=ref.logsoftmax_backward(go, lsm))

    # products, renorm, index operations, SoftMax, SpatialAveragePooling
    g = ref.rng(41)
    T = g.uniform((4, 6, 5), 0.5, 1.5)
    idx = np.array([3, 1, 6, 3], np.int64)
    src = g.normal((4, 4, 5))
    out.update(x_T=T, x_idx=idx, x_src=src, x_prodall=np.array([ref.prodall(T)]))
    for dim in (0, 1, 2):
        out["x_prod%d" % dim] = ref.prod_dim(T, dim)
        out["x_renorm%d" % dim] = np.stack([ref.renorm(T, v, dim, m) for v, m in ((1.0, 20.0), (2.0, 5.0), (3.0, 4.5))])
    out["x_select1"] = ref.index_select(T, 1, idx)
    out["x_copy1"] = ref.index_copy(T, 1, idx, src)
    out["x_fill2"] = ref.index_fill(T, 2, idx[:2], -2.5)
    z = g.normal((5, 40), 0, 2)
    sm = ref.softmax_forward(z)
    go = g.normal((5, 40))
    out.update(sm_z=z, sm_out=sm, sm_go=go, sm_gi=ref.softmax_backward(go, sm))
    img = g.normal((2, 3, 11, 13))
    out["ap_x"] = img
    for name, (kH, kW, dH, dW) in dict(ap22=(2, 2, 2, 2), ap32=(3, 3, 2, 2), ap_odd=(4, 5, 3, 2)).items():
        o = ref.sumpool_forward(img, kH, kW, dH, dW)
        go = g.normal(o.shape)
        out[name + "_cfg"] = np.array([kH, kW, dH, dW])
        out[name + "_out"], out[name + "_go"] = o, go
        out[name + "_gi"] = ref.sumpool_backward(img, go, kH, kW, dH, dW)

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_cpu.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()

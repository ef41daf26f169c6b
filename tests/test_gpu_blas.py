"""addmm / addmv / addr / gemm on the device vs the CPU oracle (TH's sequential-fp32 triple loop),
in both math modes: "fp32x3" (tcgen05 tensor cores, 3xTF32 split) and "simt" (FP32 FMA)."""
import os

import numpy as np
import pytest

from util import close, close_accumulated

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu.npz"))
MODES = ["fp32x3", "simt"]


@pytest.fixture(scope="module")
def gt():
    import mcw_cppamp_torch_b200 as m
    m.lib().THGPUInit()
    yield m
    m.set_math_mode("fp32x3")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("M,N,K", [(19, 23, 31), (128, 128, 32), (129, 65, 33), (200, 300, 100), (64, 16, 257),
                                   (1, 1, 1), (5, 1, 3), (1, 40, 7), (300, 70, 1),
                                   # two-SM tiles: 64 / 128 / 192 / 256 wide, ragged in M, N and K
                                   (257, 64, 40), (300, 190, 70), (513, 384, 96), (260, 1000, 130)])
def test_addmm_all_layouts(gt, oracle_port, mode, M, N, K):
    gt.set_math_mode(mode)
    g = oracle_port.rng(M * 1000 + N)
    t = g.normal((M, N))
    A, B = g.normal((M, K)), g.normal((K, N))
    At, Bt = g.normal((K, M)), g.normal((N, K))
    for a_np, a in ((A, gt.gpu(A)), (At.T, gt.gpu(At).t())):
        for b_np, b in ((B, gt.gpu(B)), (Bt.T, gt.gpu(Bt).t())):
            for beta, alpha in ((1.0, 1.0), (0.5, 2.0), (0.0, 1.0)):
                want = oracle_port.addmm(beta, t, alpha, a_np, b_np)
                exact = beta * t.astype(np.float64) + alpha * (a_np.astype(np.float64) @ b_np.astype(np.float64))
                r = gt.gpu(t)
                r.addmm(beta, alpha, a, b)
                close_accumulated(r.float(), want, exact, what="addmm %s" % mode)
    # transposed destination and a destination with no unit stride
    want = oracle_port.addmm(0.5, t, 2.0, A, B)
    exact = 0.5 * t.astype(np.float64) + 2.0 * (A.astype(np.float64) @ B.astype(np.float64))
    rt = gt.gpu(np.ascontiguousarray(t.T)).t()
    rt.addmm(0.5, 2.0, gt.gpu(A), gt.gpu(B))
    close_accumulated(rt.float(), want, exact, what="addmm transposed result")
    big = gt.GPUTensor(M, 2 * N).fill(0)
    rs = big.narrow(2, 1, N)                    # row stride 2N, col stride 1 -> fine; now make both non-unit
    wide = gt.GPUTensor(M, N, 2).fill(0).select(3, 1)
    wide.copy(gt.gpu(t))
    wide.addmm(0.5, 2.0, gt.gpu(A), gt.gpu(B))
    close_accumulated(wide.float(), want, exact, what="addmm strided result")
    rs.copy(gt.gpu(t))
    rs.addmm(0.5, 2.0, gt.gpu(A), gt.gpu(B))
    close_accumulated(rs.float(), want, exact, what="addmm narrowed result")


@pytest.mark.parametrize("mode", MODES)
def test_addmm_beta_zero_ignores_garbage(gt, mode):
    gt.set_math_mode(mode)
    A = np.ones((40, 8), np.float32)
    B = np.ones((8, 24), np.float32)
    r = gt.gpu(np.full((40, 24), np.nan, np.float32))
    r.addmm(0.0, 1.0, gt.gpu(A), gt.gpu(B))
    assert np.array_equal(r.float(), np.full((40, 24), 8.0, np.float32))


@pytest.mark.parametrize("mode", MODES)
def test_addmm_golden(gt, mode):
    gt.set_math_mode(mode)
    A, B, Cm, Bt = G["m_A"], G["m_B"], G["m_C"], G["m_Bt"]
    close(gt.gpu(Cm).addmm(1.0, 1.0, gt.gpu(A), gt.gpu(B)).float(), G["m_addmm"])
    close(gt.gpu(Cm).addmm(0.5, 2.0, gt.gpu(A), gt.gpu(B)).float(), G["m_addmm_b"])
    close(gt.gpu(Cm).addmm(0.5, 2.0, gt.gpu(A), gt.gpu(Bt).t()).float(), G["m_addmm_t"])


@pytest.mark.parametrize("mode", MODES)
def test_addmm_split_k_shapes(gt, oracle_port, mode):
    """Few output tiles and a long reduction: the split-K path (Linear-layer shapes, scaled down)."""
    gt.set_math_mode(mode)
    g = oracle_port.rng(77)
    M, N, K = 96, 40, 4100
    A, B, t = g.normal((M, K)), g.normal((K, N)), g.normal((M, N))
    want = oracle_port.addmm(1.0, t, 0.25, A, B)
    exact = t.astype(np.float64) + 0.25 * (A.astype(np.float64) @ B.astype(np.float64))
    got = gt.gpu(t).addmm(1.0, 0.25, gt.gpu(A), gt.gpu(B)).float()
    close_accumulated(got, want, exact, what="split-K addmm")


def test_fp32x3_is_fp32_accurate_where_one_tf32_product_is_not(gt):
    """Large common offset: a single TF32 product loses the low bits (error ~1e-3 relative), the 3-way
    split keeps them."""
    gt.set_math_mode("fp32x3")
    rs = np.random.RandomState(0)
    A = (1.0 + rs.standard_normal((128, 256)) * 1e-3).astype(np.float32)
    B = (1.0 + rs.standard_normal((256, 64)) * 1e-3).astype(np.float32)
    exact = A.astype(np.float64) @ B.astype(np.float64)
    got = gt.GPUTensor().mm(gt.gpu(A), gt.gpu(B)).float()
    assert np.abs(got - exact).max() <= 2e-6 * np.abs(exact).max()


@pytest.mark.parametrize("mode", MODES)
def test_addmv_addr(gt, oracle_port, mode):
    gt.set_math_mode(mode)
    g = oracle_port.rng(5)
    M, N = 70, 45
    A, x, y = g.normal((M, N)), g.normal((N,)), g.normal((M,))
    want = (0.5 * y.astype(np.float64) + 2.0 * (A.astype(np.float64) @ x)).astype(np.float32)
    close(gt.gpu(y).addmv(0.5, 2.0, gt.gpu(A), gt.gpu(x)).float(), want)
    At = np.ascontiguousarray(A.T)
    close(gt.gpu(y).addmv(0.5, 2.0, gt.gpu(At).t(), gt.gpu(x)).float(), want)
    u, v, R = g.normal((M,)), g.normal((N,)), g.normal((M, N))
    want = (R.astype(np.float64) + 1.5 * np.outer(u, v)).astype(np.float32)
    close(gt.gpu(R).addr(1.5, gt.gpu(u), gt.gpu(v)).float(), want)
    Rt = np.ascontiguousarray(R.T)
    close(gt.gpu(Rt).t().addr(1.5, gt.gpu(u), gt.gpu(v)).float(), want)


@pytest.mark.parametrize("mode", MODES)
def test_gemm_honours_leading_dimensions(gt, mode):
    """The raw BLAS entry point with lda/ldb/ldc larger than the matrices (the reference's kernels
    ignored them, gputorch/lib/THC/THCBlas.cpp:32,38,53)."""
    import ctypes as C
    gt.set_math_mode(mode)
    L = gt.lib()
    rs = np.random.RandomState(1)
    m, n, k, lda, ldb, ldc = 37, 21, 50, 41, 57, 45
    A = rs.standard_normal((k, lda)).astype(np.float32)   # column-major m x k with lda: A[l][i]
    B = rs.standard_normal((n, ldb)).astype(np.float32)   # column-major k x n with ldb: B[j][l]
    Cm = rs.standard_normal((n, ldc)).astype(np.float32)
    a, b, c = gt.gpu(A), gt.gpu(B), gt.gpu(Cm)
    L.THGPUBlas_gemm(b"n", b"n", m, n, k, 2.0, C.c_void_p(a.data_ptr()), lda, C.c_void_p(b.data_ptr()), ldb,
                     0.5, C.c_void_p(c.data_ptr()), ldc)
    want = Cm.copy()
    want[:, :m] = (0.5 * Cm[:, :m].astype(np.float64) +
                   2.0 * (B[:, :k].astype(np.float64) @ A[:, :m].astype(np.float64))).astype(np.float32)
    close(c.float(), want)


def test_full_size_addmm(gt, oracle_port):
    """M = N = K = 4096 (the tensor-math configuration).  The oracle's naive loop needs minutes for the
    whole product, so 48 sampled rows are checked against it and against float64; the rest through
    linearity: (A + A') B = A B + A' B within rounding."""
    gt.set_math_mode("fp32x3")
    n = 4096
    g = oracle_port.rng(4096)
    A, B = g.normal((n, n)), g.normal((n, n))
    a, b = gt.gpu(A), gt.gpu(B)
    c = gt.GPUTensor(n, n).zero().addmm(1.0, 1.0, a, b)
    got = c.float()
    rows = np.random.RandomState(0).choice(n, 48, replace=False)
    want = oracle_port.addmm(0.0, np.zeros((48, n), np.float32), 1.0, np.ascontiguousarray(A[rows]), B)
    exact = A[rows].astype(np.float64) @ B.astype(np.float64)
    close_accumulated(got[rows], want, exact, what="addmm 4096 rows")
    # transposed operands give the same product
    at = gt.gpu(np.ascontiguousarray(A.T)).t()
    ct = gt.GPUTensor(n, n).zero().addmm(1.0, 1.0, at, b).float()
    assert np.abs(ct - got).max() <= 1e-3
    # beta/alpha form on an N(0,1) C, sampled rows
    Cn = g.normal((n, n))
    got2 = gt.gpu(Cn).addmm(0.5, 2.0, a, b).float()
    close_accumulated(got2[rows], (0.5 * Cn[rows] + 2.0 * want).astype(np.float32),
                      0.5 * Cn[rows].astype(np.float64) + 2.0 * exact, what="addmm 4096 beta/alpha")
    # linearity over the whole matrix
    A2 = g.normal((n, n))
    c2 = gt.GPUTensor(n, n).zero().addmm(1.0, 1.0, gt.gpu(A2), b).float()
    c12 = gt.GPUTensor(n, n).zero().addmm(1.0, 1.0, gt.gpu(A + A2), b).float()
    assert np.abs(c12 - (got + c2)).max() <= 2e-3


@pytest.mark.parametrize("M,N,K", [(257, 64, 40), (300, 190, 70), (513, 384, 96), (260, 1000, 130), (19, 23, 31)])
def test_addmm_bf16_mode(gt, oracle_port, M, N, K):
    """Opt-in BF16 math mode: every transpose layout within BF16 accuracy (the last shape is too small for the
    BF16 engine and runs FP32-accurate)."""
    gt.set_math_mode("bf16")
    try:
        g = oracle_port.rng(M + N + K)
        t = g.normal((M, N))
        A, B = g.normal((M, K)), g.normal((K, N))
        At, Bt = g.normal((K, M)), g.normal((N, K))
        for a_np, a in ((A, gt.gpu(A)), (At.T, gt.gpu(At).t())):
            for b_np, b in ((B, gt.gpu(B)), (Bt.T, gt.gpu(Bt).t())):
                exact = 0.5 * t.astype(np.float64) + 2.0 * (a_np.astype(np.float64) @ b_np.astype(np.float64))
                r = gt.gpu(t)
                r.addmm(0.5, 2.0, a, b)
                assert np.abs(r.float() - exact).max() <= 2e-2 * np.abs(exact).max()
    finally:
        gt.set_math_mode("fp32x3")


@pytest.mark.parametrize("M,N,K,beta", [
    (19200, 512, 640, 0.0),     # 150 tiles of 256 x 256 for 74 clusters: two whole rounds + 2 tail tiles cut along k
    (19200, 512, 640, 1.0),     # the same with the accumulating epilogue (memory-side adds)
    (4096, 128, 9216, 0.0),     # fewer tiles than clusters: every tile is a tail tile (Linear at 128 rows)
    (2048, 2304, 128, 1.0),     # four k tiles per item: an outer-product-like weight gradient, epilogue-bound
    (1300, 300, 2100, 0.5),     # ragged in M, N and K; read-modify-write epilogue
])
def test_addmm_item_handout_tail_slices_and_epilogues(gt, oracle_port, M, N, K, beta):
    """Shapes that reach the persistent engine's item hand-out, its tail-only k split (tile-local partial sums
    folded by a second kernel) and its three epilogues, each against the CPU path and float64; the result must not
    depend on which cluster took which item (bit-identical across repetitions)."""
    gt.set_math_mode("fp32x3")
    g = oracle_port.rng(M + N + K)
    A, B, t = g.uniform((M, K), -1, 1), g.uniform((K, N), -1, 1), g.normal((M, N))
    exact = beta * t.astype(np.float64) + 0.5 * (A.astype(np.float64) @ B.astype(np.float64))
    ag, bg = gt.gpu(A), gt.gpu(B)
    got = gt.gpu(t).addmm(beta, 0.5, ag, bg).float()
    want = oracle_port.addmm(beta, t, 0.5, A, B)
    close_accumulated(got, want, exact, what="addmm %dx%dx%d beta %g" % (M, N, K, beta))
    for _ in range(3):
        assert np.array_equal(gt.gpu(t).addmm(beta, 0.5, ag, bg).float(), got)

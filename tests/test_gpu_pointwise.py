"""torch.GPUTensor pointwise functions, comparisons, addcmul / addcdiv and whole-tensor norms on the device vs
the CPU oracle (mcw_torch7_core/lib/TH/generic/THTensorMath.c restated in oracle/oracle.c and pinned to the
reference's own build).  Bit-exact where no transcendental function is involved; rel 1e-4 / abs 1e-5 for the
rest (single-precision device functions, 1-2 ulp from the CPU's double-precision evaluation)."""
import os

import numpy as np
import pytest

from util import POINTWISE_EXACT, close, pointwise_cases

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu.npz"))


@pytest.fixture(scope="module")
def gt():
    import mcw_cppamp_torch_b200 as m
    m.lib().THGPUInit()
    return m


def run_case(gt, name, a, b, c, v1, v2, transposed=False):
    """r:<name>(...) through the tensor methods; transposed: the first operand is a transposed view."""
    def dev(x):
        if x is None:
            return None
        if transposed:
            return gt.gpu(np.ascontiguousarray(x.T)).t()
        return gt.gpu(x)
    ta, tb, tc = dev(a), dev(b), dev(c)
    r = gt.GPUTensor()
    if name == "pow":
        r.pow(ta, v1)
    elif name == "clamp":
        r.clamp(ta, v1, v2)
    elif name == "atan2":
        r.atan2(ta, tb)
    elif name.endswith("Value"):
        getattr(r, name[:2])(ta, v1)
    elif name.endswith("Tensor"):
        getattr(r, name[:2])(ta, tb)
    elif name in ("addcmul", "addcdiv"):
        getattr(r, name)(ta, v1, tb, tc)
    else:
        getattr(r, name)(ta)
    return r.float()


@pytest.mark.parametrize("transposed", [False, True])
def test_pointwise_matches_cpu(gt, oracle_port, transposed):
    g = oracle_port.rng(31)
    X, Y = g.normal((70, 130)), g.normal((70, 130))
    for key, name, a, b, c, v1, v2 in pointwise_cases(X, Y):
        want = oracle_port.pointwise(name, a, b, c, v1, v2)
        got = run_case(gt, name, a, b, c, v1, v2, transposed)
        if key in POINTWISE_EXACT:
            assert np.array_equal(got, want), key
        else:
            close(got, want, what=key)


def test_pointwise_golden_vectors(gt):
    X, Y = G["m_X"], G["m_Y"]
    for key, name, a, b, c, v1, v2 in pointwise_cases(X, Y):
        got = run_case(gt, name, a, b, c, v1, v2)
        if key in POINTWISE_EXACT:
            assert np.array_equal(got, G["pw_" + key]), key
        else:
            close(got, G["pw_" + key], what=key)


def test_in_place_forms_and_new_result(gt, oracle_port):
    g = oracle_port.rng(32)
    X, Y = g.normal((33, 65)), g.normal((33, 65))
    t = gt.gpu(np.abs(X) + np.float32(0.5))
    want = oracle_port.pointwise("sqrt", np.abs(X) + np.float32(0.5))
    assert np.array_equal(t.sqrt().float(), want)                       # t:sqrt() in place
    m = gt.gpu(X).gt(0.0)                                               # t:gt(value) returns a new 1 / 0 tensor
    assert np.array_equal(m.float(), (X > 0).astype(np.float32))
    t = gt.gpu(X)
    t.addcmul(0.5, gt.gpu(Y), gt.gpu(Y))                                # in place on t
    assert np.array_equal(t.float(), oracle_port.pointwise("addcmul", X, Y, Y, 0.5))
    t = gt.gpu(X)
    t.addcmul(0.5, gt.gpu(Y.reshape(65, 33)), gt.gpu(Y))                # another shape, same element count
    assert np.array_equal(t.float(), oracle_port.pointwise("addcmul", X, Y, Y, 0.5))
    with pytest.raises(gt.THCError, match="sizes do not match"):
        gt.GPUTensor().atan2(gt.gpu(X), gt.gpu(Y[:, :5]))


def test_norms_match_cpu(gt, oracle_port):
    g = oracle_port.rng(33)
    X, Y = g.normal((257, 391)), g.normal((257, 391))
    x, y = gt.gpu(X), gt.gpu(Y)
    for value in (0.0, 1.0, 2.0, 3.5):
        close(np.float32(x.norm(value)), np.float32(oracle_port.normall(X, value)), what="normall %g" % value)
    # dist accumulates in a float on the CPU: over 100k terms that sum carries ~1e-4 of rounding noise itself
    for value in (1.0, 2.0, 2.5):
        close(np.float32(x.dist(y, value)), np.float32(oracle_port.dist(X, Y, value)), rtol=5e-4, what="dist %g" % value)
    close(np.float32(x.var()), np.float32(oracle_port.varall(X)), what="varall")
    close(np.float32(x.std()), np.float32(np.sqrt(oracle_port.varall(X))), what="stdall")
    xt = gt.gpu(np.ascontiguousarray(X.T)).t()                          # transposed view of the same values
    close(np.float32(xt.norm(2.0)), np.float32(oracle_port.normall(X, 2.0)), what="normall transposed")
    # the golden values of the reference itself
    gx, gy = gt.gpu(G["m_X"]), gt.gpu(G["m_Y"])
    close(np.array([gx.norm(v) for v in (0.0, 1.0, 2.0, 3.5)], np.float32), G["pw_normall"].astype(np.float32))
    close(np.array([gx.dist(gy, v) for v in (1.0, 2.0, 2.5)], np.float32), G["pw_dist"].astype(np.float32), rtol=5e-4)
    close(np.array([gx.var()], np.float32), G["pw_varall"].astype(np.float32))
    # norm along a dimension (1-based in the tensor method), plain and transposed source
    for dim in (0, 1):
        for value in (0.0, 1.0, 2.0, 3.0):
            want = oracle_port.norm_dim(X, value, dim)
            close(gt.GPUTensor().norm(x, value, dim + 1).float().reshape(-1), want, what="norm dim %d p %g" % (dim, value))
            close(gt.GPUTensor().norm(xt, value, dim + 1).float().reshape(-1), want, what="norm transposed")
        close(np.stack([gt.GPUTensor().norm(gx, v, dim + 1).float().reshape(-1) for v in (0.0, 1.0, 2.0, 3.0)]),
              G["pw_norm%d" % dim])


"""Shared helpers of the GPU parity tests."""
import numpy as np

# north-star tolerance for FP32 conv / GEMM outputs and gradients
RTOL, ATOL = 1e-4, 1e-5


def close(actual, desired, rtol=RTOL, atol=ATOL, what=""):
    actual, desired = np.asarray(actual), np.asarray(desired)
    assert actual.shape == desired.shape, (what, actual.shape, desired.shape)
    err = np.abs(actual.astype(np.float64) - desired.astype(np.float64))
    bound = atol + rtol * np.abs(desired.astype(np.float64))
    bad = err > bound
    if bad.any():
        i = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError("%s: %d of %d outside |d| <= %g + %g|ref|; worst at %s: got %r want %r" %
                             (what, bad.sum(), bad.size, atol, rtol, i, actual[i], desired[i]))


def close_accumulated(actual, oracle, exact64, rtol=RTOL, atol=ATOL, what=""):
    """For long fp32 reductions: the oracle's own sequential-fp32 rounding noise (measured against a
    float64 evaluation) can exceed the elementwise bound near zero, so the device result must sit
    within the bound of the float64 value, or within the bound widened by the oracle's own error."""
    err_dev = np.abs(actual.astype(np.float64) - exact64)
    err_orc = np.abs(oracle.astype(np.float64) - exact64)
    bound = atol + rtol * np.abs(exact64)
    ok = (err_dev <= bound) | (np.abs(actual.astype(np.float64) - oracle) <= bound + err_orc)
    assert ok.all(), "%s: %d of %d elements outside tolerance (max dev err %g, max oracle err %g)" % (
        what, (~ok).sum(), ok.size, err_dev.max(), err_orc.max())

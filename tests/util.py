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
    """For fp32 reductions over many terms.  The CPU oracle's own rounding noise (its distance from a
    float64 evaluation of the same sum) routinely exceeds abs 1e-5 for near-zero outputs, so two correct
    fp32 implementations with different summation orders cannot agree elementwise at that bound.  What
    is asserted instead: the device result lies within the bound of the float64 value, widened by the
    oracle's worst own error on this very problem (the device may not be less accurate than the
    oracle by more than the tolerance)."""
    exact64 = np.asarray(exact64, dtype=np.float64)
    err_dev = np.abs(np.asarray(actual, dtype=np.float64) - exact64)
    err_orc = np.abs(np.asarray(oracle, dtype=np.float64) - exact64)
    bound = atol + rtol * np.abs(exact64) + err_orc.max()
    ok = err_dev <= bound
    assert ok.all(), "%s: %d of %d elements outside tolerance (max dev err %g, max oracle err %g)" % (
        what, (~ok).sum(), ok.size, err_dev.max(), err_orc.max())


# ---- float64 evaluations of the convolution passes (the "true" values both the CPU oracle and the
# device approximate in fp32) ----
def _windows(x, kH, kW, dH, dW, pad):
    xp = np.pad(x.astype(np.float64), ((0, 0), (0, 0), (pad, pad), (pad, pad)))
    win = np.lib.stride_tricks.sliding_window_view(xp, (kH, kW), axis=(2, 3))
    return win[:, :, ::dH, ::dW]          # [N, C, oH, oW, kH, kW]


def conv_exact(x, w, b, kH, kW, dH, dW, pad):
    K, C = w.shape[0], x.shape[1]
    win = _windows(x, kH, kW, dH, dW, pad)
    return np.einsum("nchwij,kcij->nkhw", win, w.reshape(K, C, kH, kW).astype(np.float64), optimize=True) + \
        b.astype(np.float64)[None, :, None, None]


def conv_grad_weight_exact(x, go, kH, kW, dH, dW, pad):
    win = _windows(x, kH, kW, dH, dW, pad)
    gw = np.einsum("nchwij,nkhw->kcij", win, go.astype(np.float64), optimize=True)
    return gw.reshape(gw.shape[0], -1), go.astype(np.float64).sum(axis=(0, 2, 3))


def conv_grad_input_exact(go, w, in_shape, kH, kW, dH, dW, pad):
    N, C, H, W = in_shape
    K = w.shape[0]
    oH, oW = go.shape[2:]
    w4 = w.reshape(K, C, kH, kW).astype(np.float64)
    g = np.zeros((N, C, H + 2 * pad, W + 2 * pad))
    go64 = go.astype(np.float64)
    for i in range(kH):
        for j in range(kW):
            g[:, :, i:i + oH * dH:dH, j:j + oW * dW:dW] += np.einsum("nkhw,kc->nchw", go64, w4[:, :, i, j])
    return g[:, :, pad:pad + H, pad:pad + W]


def pointwise_cases(X, Y):
    """(key, name, a, b, c, v1, v2) for every pointwise operation of the tensor-math surface, with inputs
    inside each function's domain.  The inputs are made from X and Y with exact operations only (abs, clip,
    scaling by powers of two), so that they are the same numbers on every machine."""
    X, Y = np.ascontiguousarray(X, np.float32), np.ascontiguousarray(Y, np.float32)
    pos = np.abs(X) + np.float32(0.125)
    unit = np.clip(X * np.float32(0.5), np.float32(-0.96875), np.float32(0.96875))
    half = np.round(X * 4) / np.float32(4)            # many exact halves and integers: round / ceil / floor / eq
    halfy = np.round(Y * 4) / np.float32(4)
    nz = np.where(np.abs(Y) < 0.25, np.float32(0.5), Y)
    cases = []
    for name in ("exp", "cos", "cosh", "sin", "sinh", "tan", "atan", "tanh", "abs", "sign"):
        cases.append((name, name, X, None, None, 0.0, 0.0))
    for name in ("log", "log1p", "sqrt"):
        cases.append((name, name, pos, None, None, 0.0, 0.0))
    for name in ("acos", "asin"):
        cases.append((name, name, unit, None, None, 0.0, 0.0))
    for name in ("ceil", "floor", "round"):
        cases.append((name, name, half, None, None, 0.0, 0.0))
    cases.append(("pow_frac", "pow", pos, None, None, 1.75, 0.0))
    cases.append(("pow_int", "pow", X, None, None, 3.0, 0.0))
    cases.append(("clamp", "clamp", X, None, None, -0.5, 0.75))
    cases.append(("atan2", "atan2", X, Y, None, 0.0, 0.0))
    for op in ("lt", "gt", "le", "ge", "eq", "ne"):
        cases.append((op + "Value", op + "Value", half, None, None, 0.25, 0.0))
        cases.append((op + "Tensor", op + "Tensor", half, halfy, None, 0.0, 0.0))
    cases.append(("addcmul", "addcmul", X, Y, pos, 0.3, 0.0))
    cases.append(("addcdiv", "addcdiv", X, Y, nz, -1.7, 0.0))
    return cases


# results that every correct implementation gives bit for bit (no transcendental function involved)
POINTWISE_EXACT = {"abs", "sign", "sqrt", "ceil", "floor", "round", "clamp", "addcmul", "addcdiv"} | {
    op + kind for op in ("lt", "gt", "le", "ge", "eq", "ne") for kind in ("Value", "Tensor")}

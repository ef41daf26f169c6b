"""Shared helpers of the GPU parity tests."""
import numpy as np

# north-star tolerance for FP32 conv / GEMM outputs and gradients
RTOL, ATOL = 1e-4, 1e-5

# One line per comparison of a long FP32 reduction: how many elements miss the LITERAL bound
# |device - cpu| <= 1e-5 + 1e-4 |cpu| and by how much, next to the outcome of the widened bound the test asserts.
# tests/conftest.py prints the lines at the end of the run, so the tolerance argument can be read off the log.
PARITY_REPORT = []


def report_literal_bound(what, actual, cpu, outcome, rtol=RTOL, atol=ATOL):
    a, c = np.asarray(actual, np.float64), np.asarray(cpu, np.float64)
    err = np.abs(a - c)
    bound = atol + rtol * np.abs(c)
    miss = err > bound
    worst = float((err / bound).max()) if err.size else 0.0
    PARITY_REPORT.append("%-58s %9d elements, %7d outside 1e-5 + 1e-4|cpu| (worst %.2f x bound, max |d| %.3g); asserted: %s" % (
        what[:58], err.size, int(miss.sum()), worst, float(err.max()) if err.size else 0.0, outcome))


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
    report_literal_bound(what or "accumulated", actual, oracle,
                         "within bound of float64 widened by the oracle's own worst error %.3g (device worst %.3g): %s" % (
                             err_orc.max(), err_dev.max(), "pass" if ok.all() else "FAIL"), rtol, atol)
    assert ok.all(), "%s: %d of %d elements outside tolerance (max dev err %g, max oracle err %g)" % (
        what, (~ok).sum(), ok.size, err_dev.max(), err_orc.max())


def close_scaled(actual, cpu, what="", rtol=RTOL, atol=ATOL):
    """Gradients of a whole network: sums of many FP32 products of both signs, where entries near zero carry the
    CPU's own summation noise.  Asserted against the tensor's scale, |d| <= 1e-5 + 1e-4 max|cpu|; the count of
    elements outside the literal element-wise bound goes on the parity report."""
    a, c = np.asarray(actual, np.float64), np.asarray(cpu, np.float64)
    assert a.shape == c.shape, (what, a.shape, c.shape)
    scale = np.abs(c).max() if c.size else 0.0
    worst = np.abs(a - c).max() if c.size else 0.0
    ok = worst <= atol + rtol * scale
    report_literal_bound(what, a, c, "max |d| %.3g <= 1e-5 + 1e-4 * max|cpu| (%.3g): %s" % (worst, scale, "pass" if ok else "FAIL"),
                         rtol, atol)
    assert ok, (what, worst, scale)


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


# ---- a whole classifier step on the CPU path (plain-C restatement), layer list given by the caller
def cpu_classifier_step(port, convs, fcs, x, labels, params):
    """Forward, ClassNLL loss and backward of conv/ReLU/[max-pool] blocks followed by Linear/ReLU layers and
    LogSoftMax, every operator through `port`.  convs: (nIn, nOut, k, stride, pad, pool) with pool None or
    (k, stride); params: [(weight 2-D, bias)] conv layers first.  Returns (loss, [(gradWeight, gradBias)]) in
    layer order; the first conv computes no gradInput."""
    n = x.shape[0]
    acts, cur = [], x
    for (ci, co, k, s, p, pool), (w, b) in zip(convs, params):
        c = port.conv_forward(cur, w, b, k, k, s, s, p)
        r = port.threshold_forward(c)
        ind = None
        nxt = r
        if pool:
            nxt, ind = port.maxpool_forward(r, pool[0], pool[0], pool[1], pool[1])
        acts.append((cur, c, r, ind))
        cur = nxt
    h = cur.reshape(n, -1)
    fc_acts = []
    fc_params = params[len(convs):]
    for i, (w, b) in enumerate(fc_params):
        z = port.addmm(1.0, np.tile(b, (n, 1)).astype(np.float32), 1.0, h, w.T)
        fc_acts.append((h, z))
        h = port.threshold_forward(z) if i < len(fc_params) - 1 else z
    lsm = port.logsoftmax_forward(h)
    loss = port.classnll_forward(lsm, labels)
    g = port.logsoftmax_backward(port.classnll_backward(labels, lsm.shape), lsm)
    grads = []
    for i in range(len(fc_params) - 1, -1, -1):
        hin, z = fc_acts[i]
        w, b = fc_params[i]
        if i < len(fc_params) - 1:
            g = port.threshold_backward(z, g)
        gw = port.addmm(0.0, np.zeros_like(w), 1.0, np.ascontiguousarray(g.T), hin)
        grads.append((gw, g.sum(0, dtype=np.float32)))
        g = port.addmm(0.0, np.zeros_like(hin), 1.0, g, w)
    g = g.reshape(cur.shape)
    for li in range(len(convs) - 1, -1, -1):
        inp, c, r, ind = acts[li]
        ci, co, k, s, p, pool = convs[li]
        w, b = params[li]
        if pool:
            g = port.maxpool_backward(g, ind, r.shape, pool[1], pool[1])
        g = port.threshold_backward(c, g)
        gw, gb = np.zeros_like(w), np.zeros_like(b)
        port.conv_acc_grad(inp, g, gw, gb, 1.0, k, k, s, s, p)
        grads.append((gw, gb))
        if li > 0:
            g = port.conv_grad_input(g, w, inp.shape, k, k, s, s, p)
    return float(loss), grads[::-1]

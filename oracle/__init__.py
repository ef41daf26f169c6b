"""TEST INFRASTRUCTURE ONLY: ctypes front-ends for the two CPU checkers.

* ``port``  -- ``liboracle.so`` built from ``oracle.c`` beside this file: our plain-C restatement
  of the reference's CPU path.  Always buildable (gcc only).
* ``ref``   -- ``_ref/liboracle_ref.so``: the reference's OWN TH + nn CPU sources compiled by the
  Makefile's ``ref`` target (needs the reference tree at build time; the built file travels).

Only tests, the smoke run and the bench's CPU-baseline / reference legs may import this module.
The product package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT_SO = os.path.join(_HERE, "liboracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "liboracle_ref.so")

_fp = C.POINTER(C.c_float)
_lp = C.POINTER(C.c_long)


def reference_root():
    """Where the reference tree lies: $ORACLE_REF, else `reference_path` of BASELINE.json beside this package;
    None when neither names an existing directory (the prebuilt _ref library, if any, is then used as it is)."""
    cand = os.environ.get("ORACLE_REF")
    if not cand:
        try:
            import json
            with open(os.path.join(os.path.dirname(_HERE), "BASELINE.json")) as fh:
                cand = json.load(fh).get("reference_path")
        except (OSError, ValueError):
            cand = None
    return cand if cand and os.path.isdir(cand) else None


def build(verbose=False):
    """Compile the port (always) and the reference build (when its tree is mounted)."""
    out = None if verbose else subprocess.DEVNULL
    subprocess.check_call(["make", "-s", "-C", _HERE, "port"], stdout=out)
    ref = reference_root()
    if ref:
        subprocess.call(["make", "-s", "-C", _HERE, "ref", "REF=" + ref], stdout=out, stderr=out)


def _f(a):
    assert a.dtype == np.float32
    return a.ctypes.data_as(_fp)


def _cf(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def conv_out_size(H, W, kH, kW, dH, dW, pad):
    return (H + 2 * pad - kH) // dH + 1, (W + 2 * pad - kW) // dW + 1


# operation codes of orc_pointwise (oracle.c), by position
ORC_POINTWISE_NAMES = ["log", "log1p", "exp", "cos", "acos", "cosh", "sin", "asin", "sinh", "tan", "atan", "tanh",
                       "sqrt", "ceil", "floor", "abs", "sign", "round", "pow", "clamp", "atan2",
                       "ltValue", "gtValue", "leValue", "geValue", "eqValue", "neValue",
                       "ltTensor", "gtTensor", "leTensor", "geTensor", "eqTensor", "neTensor", "addcmul", "addcdiv"]


class _Port:
    """Numpy-in / numpy-out wrappers over oracle.c."""

    def __init__(self):
        self._lib = None

    @property
    def lib(self):
        if self._lib is None:
            if not os.path.exists(_PORT_SO):
                build()
            L = C.CDLL(_PORT_SO)
            L.orc_rng_new.restype = C.c_void_p
            L.orc_rng_new.argtypes = [C.c_ulong]
            L.orc_rng_free.argtypes = [C.c_void_p]
            L.orc_rng_uniform.argtypes = [C.c_void_p, _fp, C.c_long, C.c_double, C.c_double]
            L.orc_rng_normal.argtypes = [C.c_void_p, _fp, C.c_long, C.c_double, C.c_double]
            l10 = [C.c_long] * 10
            L.orc_conv_mm_forward.argtypes = [_fp, _fp, _fp, _fp] + l10
            L.orc_conv_mm_grad_input.argtypes = [_fp, _fp, _fp] + l10
            L.orc_conv_mm_acc_grad.argtypes = [_fp, _fp, _fp, _fp, C.c_float] + l10
            L.orc_maxpool_forward.argtypes = [_fp, _fp, _fp] + [C.c_long] * 7
            L.orc_maxpool_backward.argtypes = [_fp, _fp, _fp] + [C.c_long] * 7
            L.orc_threshold_forward.argtypes = [_fp, _fp, C.c_long, C.c_double, C.c_double]
            L.orc_threshold_backward.argtypes = [_fp, _fp, _fp, C.c_long, C.c_double]
            L.orc_add.argtypes = [_fp, C.c_long, C.c_long, _fp, C.c_long, C.c_long, C.c_float,
                                  C.c_long, C.c_long]
            L.orc_cadd.argtypes = [_fp, C.c_long, C.c_long, _fp, C.c_long, C.c_long, C.c_float,
                                   _fp, C.c_long, C.c_long, C.c_long, C.c_long]
            L.orc_cmul.argtypes = [_fp, C.c_long, C.c_long, _fp, C.c_long, C.c_long,
                                   _fp, C.c_long, C.c_long, C.c_long, C.c_long]
            L.orc_sumall.restype = C.c_double
            L.orc_sumall.argtypes = [_fp] + [C.c_long] * 4
            L.orc_maxall.restype = C.c_float
            L.orc_maxall.argtypes = [_fp] + [C.c_long] * 4
            L.orc_sum_dim.argtypes = [_fp, _fp] + [C.c_long] * 4 + [C.c_int]
            L.orc_max_dim.argtypes = [_fp, _lp, _fp] + [C.c_long] * 4 + [C.c_int]
            L.orc_addmm.argtypes = [_fp, C.c_long, C.c_long, C.c_float, _fp, C.c_long, C.c_long,
                                    C.c_float, _fp, C.c_long, C.c_long, _fp, C.c_long, C.c_long,
                                    C.c_long, C.c_long, C.c_long]
            L.orc_pointwise.argtypes = [C.c_int, _fp, _fp, _fp, _fp, C.c_long, C.c_float, C.c_float]
            L.orc_normall.restype = C.c_double
            L.orc_normall.argtypes = [_fp, C.c_long, C.c_float]
            L.orc_dist.restype = C.c_double
            L.orc_dist.argtypes = [_fp, _fp, C.c_long, C.c_float]
            L.orc_varall.restype = C.c_double
            L.orc_varall.argtypes = [_fp, C.c_long]
            L.orc_norm_dim.argtypes = [_fp, _fp, C.c_long, C.c_long, C.c_float, C.c_int]
            L.orc_prodall.restype = C.c_double
            L.orc_prodall.argtypes = [_fp, C.c_long]
            L.orc_prod_dim.argtypes = [_fp, _fp] + [C.c_long] * 3
            L.orc_renorm.argtypes = [_fp, _fp] + [C.c_long] * 3 + [C.c_float, C.c_float]
            L.orc_index_select.argtypes = [_fp, _fp, _lp] + [C.c_long] * 4
            L.orc_index_copy.argtypes = [_fp, _fp, _lp] + [C.c_long] * 4
            L.orc_index_fill.argtypes = [_fp, _lp] + [C.c_long] * 4 + [C.c_float]
            L.orc_softmax_forward.argtypes = [_fp, _fp, C.c_long, C.c_long]
            L.orc_softmax_backward.argtypes = [_fp, _fp, _fp, C.c_long, C.c_long]
            L.orc_sumpool_forward.argtypes = [_fp, _fp] + [C.c_long] * 3 + [C.c_int] * 4
            L.orc_sumpool_backward.argtypes = [_fp, _fp] + [C.c_long] * 3 + [C.c_int] * 4
            L.orc_logsoftmax_forward.argtypes = [_fp, _fp, C.c_long, C.c_long]
            L.orc_logsoftmax_backward.argtypes = [_fp, _fp, _fp, C.c_long, C.c_long]
            L.orc_classnll_forward.restype = C.c_double
            L.orc_classnll_forward.argtypes = [_fp, _fp, C.c_long, C.c_long]
            L.orc_classnll_backward.argtypes = [_fp, _fp, C.c_long, C.c_long]
            self._lib = L
        return self._lib

    # ---- seeded inputs (TH's MT19937 stream) ----
    class Rng:
        def __init__(self, port, seed):
            self._p = port
            self._g = port.lib.orc_rng_new(seed)

        def uniform(self, shape, a, b):
            out = np.empty(shape, np.float32)
            self._p.lib.orc_rng_uniform(self._g, _f(out), out.size, a, b)
            return out

        def normal(self, shape, mean=0.0, std=1.0):
            out = np.empty(shape, np.float32)
            self._p.lib.orc_rng_normal(self._g, _f(out), out.size, mean, std)
            return out

        def __del__(self):
            try:
                self._p.lib.orc_rng_free(self._g)
            except Exception:
                pass

    def rng(self, seed):
        return _Port.Rng(self, seed)

    # ---- nn ----
    def conv_forward(self, x, w, b, kH, kW, dH, dW, pad):
        x, w, b = _cf(x), _cf(w), _cf(b)
        N, Cc, H, W = x.shape
        K = w.shape[0]
        oH, oW = conv_out_size(H, W, kH, kW, dH, dW, pad)
        out = np.empty((N, K, oH, oW), np.float32)
        self.lib.orc_conv_mm_forward(_f(x), _f(w), _f(b), _f(out), N, Cc, H, W, K, kH, kW, dH, dW, pad)
        return out

    def conv_grad_input(self, go, w, in_shape, kH, kW, dH, dW, pad):
        go, w = _cf(go), _cf(w)
        N, Cc, H, W = in_shape
        K = w.shape[0]
        gi = np.empty(in_shape, np.float32)
        self.lib.orc_conv_mm_grad_input(_f(go), _f(w), _f(gi), N, Cc, H, W, K, kH, kW, dH, dW, pad)
        return gi

    def conv_acc_grad(self, x, go, gw, gb, scale, kH, kW, dH, dW, pad):
        """Accumulates into gw/gb (float32 contiguous arrays) in place."""
        x, go = _cf(x), _cf(go)
        N, Cc, H, W = x.shape
        K = gw.shape[0]
        self.lib.orc_conv_mm_acc_grad(_f(x), _f(go), _f(gw), _f(gb), scale, N, Cc, H, W, K, kH, kW,
                                      dH, dW, pad)

    def maxpool_forward(self, x, kH, kW, dH, dW):
        x = _cf(x)
        lead, (H, W) = x.shape[:-2], x.shape[-2:]
        NC = int(np.prod(lead))
        oH, oW = (H - kH) // dH + 1, (W - kW) // dW + 1
        out = np.empty(lead + (oH, oW), np.float32)
        ind = np.empty((2,) + lead + (oH, oW), np.float32)
        self.lib.orc_maxpool_forward(_f(x), _f(out), _f(ind), NC, H, W, kH, kW, dH, dW)
        return out, ind

    def maxpool_backward(self, go, ind, in_shape, dH, dW):
        go, ind = _cf(go), _cf(ind)
        H, W = in_shape[-2:]
        NC = int(np.prod(in_shape[:-2]))
        oH, oW = go.shape[-2:]
        gi = np.empty(in_shape, np.float32)
        self.lib.orc_maxpool_backward(_f(go), _f(ind), _f(gi), NC, H, W, oH, oW, dH, dW)
        return gi

    def threshold_forward(self, x, th=0.0, val=0.0):
        x = _cf(x)
        out = np.empty_like(x)
        self.lib.orc_threshold_forward(_f(x), _f(out), x.size, th, val)
        return out

    def threshold_backward(self, x, go, th=0.0):
        x, go = _cf(x), _cf(go)
        gi = np.empty_like(x)
        self.lib.orc_threshold_backward(_f(x), _f(go), _f(gi), x.size, th)
        return gi

    # ---- tensor math on (possibly transposed) 2-D float32 views ----
    @staticmethod
    def _v(a):
        assert a.dtype == np.float32 and a.ndim == 2
        return _f(a), a.strides[0] // 4, a.strides[1] // 4

    def add(self, t, value):
        r = np.empty(t.shape, np.float32)
        self.lib.orc_add(*self._v(r), *self._v(t), value, *t.shape)
        return r

    def cadd(self, t, value, s):
        r = np.empty(t.shape, np.float32)
        self.lib.orc_cadd(*self._v(r), *self._v(t), value, *self._v(s), *t.shape)
        return r

    def cmul(self, t, s):
        r = np.empty(t.shape, np.float32)
        self.lib.orc_cmul(*self._v(r), *self._v(t), *self._v(s), *t.shape)
        return r

    def pointwise(self, name, a, b=None, c=None, v1=0.0, v2=0.0):
        """r = name(a[, b[, c]]) element by element on contiguous arrays; names: ORC_POINTWISE_NAMES."""
        a = np.ascontiguousarray(a, np.float32)
        b = a if b is None else np.ascontiguousarray(b, np.float32)
        c = a if c is None else np.ascontiguousarray(c, np.float32)
        r = np.empty(a.shape, np.float32)
        self.lib.orc_pointwise(ORC_POINTWISE_NAMES.index(name), _f(r), _f(a), _f(b), _f(c), a.size, v1, v2)
        return r

    def normall(self, t, value):
        t = np.ascontiguousarray(t, np.float32)
        return self.lib.orc_normall(_f(t), t.size, value)

    def dist(self, a, b, value):
        a, b = np.ascontiguousarray(a, np.float32), np.ascontiguousarray(b, np.float32)
        return self.lib.orc_dist(_f(a), _f(b), a.size, value)

    def varall(self, t):
        t = np.ascontiguousarray(t, np.float32)
        return self.lib.orc_varall(_f(t), t.size)

    def norm_dim(self, t, value, dim):
        t = np.ascontiguousarray(t, np.float32)
        r = np.empty(t.shape[1] if dim == 0 else t.shape[0], np.float32)
        self.lib.orc_norm_dim(_f(r), _f(t), t.shape[0], t.shape[1], value, dim)
        return r

    # ---- [outer][D][inner] blocks of a contiguous array around dimension `dim` (0-based) ----
    @staticmethod
    def _block(shape, dim):
        outer = int(np.prod(shape[:dim], dtype=np.int64))
        inner = int(np.prod(shape[dim + 1:], dtype=np.int64))
        return outer, shape[dim], inner

    def prodall(self, t):
        t = np.ascontiguousarray(t, np.float32)
        return self.lib.orc_prodall(_f(t), t.size)

    def prod_dim(self, t, dim):
        t = np.ascontiguousarray(t, np.float32)
        shape = list(t.shape); shape[dim] = 1
        r = np.empty(shape, np.float32)
        self.lib.orc_prod_dim(_f(r), _f(t), *self._block(t.shape, dim))
        return r

    def renorm(self, t, value, dim, maxnorm):
        t = np.ascontiguousarray(t, np.float32)
        r = np.empty_like(t)
        self.lib.orc_renorm(_f(r), _f(t), *self._block(t.shape, dim), value, maxnorm)
        return r

    def index_select(self, t, dim, idx):
        t = np.ascontiguousarray(t, np.float32)
        idx = np.ascontiguousarray(idx, np.int64)
        shape = list(t.shape); shape[dim] = idx.size
        r = np.empty(shape, np.float32)
        outer, D, inner = self._block(t.shape, dim)
        self.lib.orc_index_select(_f(r), _f(t), idx.ctypes.data_as(_lp), outer, D, idx.size, inner)
        return r

    def index_copy(self, res, dim, idx, src):
        r = np.ascontiguousarray(res, np.float32).copy()
        src = np.ascontiguousarray(src, np.float32)
        idx = np.ascontiguousarray(idx, np.int64)
        outer, D, inner = self._block(r.shape, dim)
        self.lib.orc_index_copy(_f(r), _f(src), idx.ctypes.data_as(_lp), outer, D, idx.size, inner)
        return r

    def index_fill(self, res, dim, idx, val):
        r = np.ascontiguousarray(res, np.float32).copy()
        idx = np.ascontiguousarray(idx, np.int64)
        outer, D, inner = self._block(r.shape, dim)
        self.lib.orc_index_fill(_f(r), idx.ctypes.data_as(_lp), outer, D, idx.size, inner, val)
        return r

    def softmax_forward(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty_like(x)
        self.lib.orc_softmax_forward(_f(x), _f(out), x.shape[0] if x.ndim == 2 else 1, x.shape[-1])
        return out

    def softmax_backward(self, go, out):
        go, out = np.ascontiguousarray(go, np.float32), np.ascontiguousarray(out, np.float32)
        gi = np.empty_like(out)
        self.lib.orc_softmax_backward(_f(go), _f(out), _f(gi), out.shape[0] if out.ndim == 2 else 1, out.shape[-1])
        return gi

    def sumpool_forward(self, x, kH, kW, dH, dW):
        x = np.ascontiguousarray(x, np.float32)
        H, W = x.shape[-2:]
        out = np.empty(x.shape[:-2] + ((H - kH) // dH + 1, (W - kW) // dW + 1), np.float32)
        self.lib.orc_sumpool_forward(_f(x), _f(out), x.size // (H * W), H, W, kH, kW, dH, dW)
        return out

    def sumpool_backward(self, go, in_shape, kH, kW, dH, dW):
        go = np.ascontiguousarray(go, np.float32)
        H, W = in_shape[-2:]
        gi = np.empty(in_shape, np.float32)
        self.lib.orc_sumpool_backward(_f(go), _f(gi), gi.size // (H * W), H, W, kH, kW, dH, dW)
        return gi

    def sumall(self, t):
        return self.lib.orc_sumall(*self._v(t), *t.shape)

    def maxall(self, t):
        return self.lib.orc_maxall(*self._v(t), *t.shape)

    def sum_dim(self, t, dim):
        r = np.empty(t.shape[1 - dim], np.float32)
        self.lib.orc_sum_dim(_f(r), *self._v(t), *t.shape, dim)
        return r

    def max_dim(self, t, dim):
        r = np.empty(t.shape[1 - dim], np.float32)
        idx = np.empty(t.shape[1 - dim], np.int64)
        self.lib.orc_max_dim(_f(r), idx.ctypes.data_as(_lp), *self._v(t), *t.shape, dim)
        return r, idx

    def addmm(self, beta, t, alpha, m1, m2):
        M, K = m1.shape
        N = m2.shape[1]
        r = np.empty((M, N), np.float32)
        self.lib.orc_addmm(*self._v(r), beta, *self._v(t), alpha, *self._v(m1), *self._v(m2), M, N, K)
        return r

    def logsoftmax_forward(self, x):
        x = _cf(x)
        out = np.empty_like(x)
        self.lib.orc_logsoftmax_forward(_f(x), _f(out), *x.shape)
        return out

    def logsoftmax_backward(self, go, out):
        go, out = _cf(go), _cf(out)
        gi = np.empty_like(out)
        self.lib.orc_logsoftmax_backward(_f(go), _f(out), _f(gi), *out.shape)
        return gi

    def classnll_forward(self, x, target):
        x, target = _cf(x), _cf(target)
        return self.lib.orc_classnll_forward(_f(x), _f(target), *x.shape)

    def classnll_backward(self, target, shape):
        target = _cf(target)
        gi = np.empty(shape, np.float32)
        self.lib.orc_classnll_backward(_f(target), _f(gi), *shape)
        return gi


port = _Port()


class _Ref:
    """The reference's own compiled CPU code (TH tensors + unmodified nn kernels)."""

    def __init__(self):
        self._lib = None

    def available(self):
        return os.path.exists(_REF_SO)

    @property
    def lib(self):
        if self._lib is None:
            if not self.available():
                raise RuntimeError("reference build %s is missing (make -C oracle ref)" % _REF_SO)
            L = C.CDLL(_REF_SO)
            vp = C.c_void_p
            for name in ("THFloatTensor_new", "THFloatTensor_newWithSize1d", "THFloatTensor_newWithSize2d",
                         "THFloatTensor_newWithSize3d", "THFloatTensor_newWithSize4d",
                         "THFloatTensor_newTranspose", "THFloatTensor_data", "THLongTensor_new",
                         "THLongTensor_data", "THGenerator_new", "oref_state_new"):
                getattr(L, name).restype = vp
            L.THFloatTensor_newWithSize1d.argtypes = [C.c_long]
            L.THFloatTensor_newWithSize2d.argtypes = [C.c_long] * 2
            L.THFloatTensor_newWithSize3d.argtypes = [C.c_long] * 3
            L.THFloatTensor_newWithSize4d.argtypes = [C.c_long] * 4
            L.THFloatTensor_newTranspose.argtypes = [vp, C.c_int, C.c_int]
            L.THFloatTensor_data.argtypes = [vp]
            L.THLongTensor_data.argtypes = [vp]
            L.THFloatTensor_free.argtypes = [vp]
            L.THLongTensor_free.argtypes = [vp]
            L.THFloatTensor_nDimension.argtypes = [vp]
            L.THFloatTensor_size.argtypes = [vp, C.c_int]
            L.THFloatTensor_size.restype = C.c_long
            L.THLongTensor_size.argtypes = [vp, C.c_int]
            L.THLongTensor_size.restype = C.c_long
            L.THLongTensor_nDimension.argtypes = [vp]
            L.THFloatTensor_nElement.argtypes = [vp]
            L.THFloatTensor_nElement.restype = C.c_long
            L.THRandom_manualSeed.argtypes = [vp, C.c_ulong]
            L.THGenerator_free.argtypes = [vp]
            L.THFloatTensor_uniform.argtypes = [vp, vp, C.c_double, C.c_double]
            L.THFloatTensor_normal.argtypes = [vp, vp, C.c_double, C.c_double]
            L.THFloatTensor_add.argtypes = [vp, vp, C.c_float]
            L.THFloatTensor_cadd.argtypes = [vp, vp, C.c_float, vp]
            L.THFloatTensor_cmul.argtypes = [vp, vp, vp]
            L.THFloatTensor_sumall.argtypes = [vp]
            L.THFloatTensor_sumall.restype = C.c_double
            L.THFloatTensor_maxall.argtypes = [vp]
            L.THFloatTensor_maxall.restype = C.c_float
            L.THFloatTensor_sum.argtypes = [vp, vp, C.c_int]
            L.THFloatTensor_max.argtypes = [vp, vp, vp, C.c_int]
            L.THFloatTensor_addmm.argtypes = [vp, C.c_float, vp, C.c_float, vp, vp]
            for name in ORC_POINTWISE_NAMES[:18]:
                getattr(L, "THFloatTensor_" + name).argtypes = [vp, vp]
            L.THFloatTensor_pow.argtypes = [vp, vp, C.c_float]
            L.THFloatTensor_clamp.argtypes = [vp, vp, C.c_float, C.c_float]
            L.THFloatTensor_atan2.argtypes = [vp, vp, vp]
            for name in ("lt", "gt", "le", "ge", "eq", "ne"):
                getattr(L, "THFloatTensor_%sValueT" % name).argtypes = [vp, vp, C.c_float]
                getattr(L, "THFloatTensor_%sTensorT" % name).argtypes = [vp, vp, vp]
            L.THFloatTensor_addcmul.argtypes = [vp, vp, C.c_float, vp, vp]
            L.THFloatTensor_addcdiv.argtypes = [vp, vp, C.c_float, vp, vp]
            for name in ("normall", "dist", "varall"):
                getattr(L, "THFloatTensor_" + name).restype = C.c_double
            L.THFloatTensor_normall.argtypes = [vp, C.c_float]
            L.THFloatTensor_dist.argtypes = [vp, vp, C.c_float]
            L.THFloatTensor_varall.argtypes = [vp]
            L.THFloatTensor_norm.argtypes = [vp, vp, C.c_float, C.c_int]
            L.THFloatTensor_zero.argtypes = [vp]
            L.THFloatTensor_resizeAs.argtypes = [vp, vp]
            L.THFloatTensor_prodall.argtypes = [vp]
            L.THFloatTensor_prodall.restype = C.c_double
            L.THFloatTensor_prod.argtypes = [vp, vp, C.c_int]
            L.THFloatTensor_renorm.argtypes = [vp, vp, C.c_float, C.c_int, C.c_float]
            L.THFloatTensor_indexSelect.argtypes = [vp, vp, C.c_int, vp]
            L.THFloatTensor_indexCopy.argtypes = [vp, C.c_int, vp, vp]
            L.THFloatTensor_indexFill.argtypes = [vp, C.c_int, vp, C.c_float]
            L.THLongTensor_newWithSize1d.argtypes = [C.c_long]
            L.THLongTensor_newWithSize1d.restype = vp
            L.oref_state_free.argtypes = [vp]
            L.oref_errmsg.argtypes = [vp]
            L.oref_errmsg.restype = C.c_char_p
            L.oref_set_num.argtypes = [vp, C.c_char_p, C.c_double]
            L.oref_set_ud.argtypes = [vp, C.c_char_p, vp]
            L.oref_set_arg_ud.argtypes = [vp, C.c_int, vp]
            L.oref_set_arg_num.argtypes = [vp, C.c_int, C.c_double]
            L.oref_call.argtypes = [vp, C.c_char_p]
            self._lib = L
        return self._lib

    # ---- TH tensors <-> numpy ----
    def tensor(self, a=None):
        """New contiguous THFloatTensor holding a copy of ``a`` (or an empty tensor)."""
        L = self.lib
        if a is None:
            return L.THFloatTensor_new()
        a = np.ascontiguousarray(a, np.float32)
        ctor = {1: L.THFloatTensor_newWithSize1d, 2: L.THFloatTensor_newWithSize2d,
                3: L.THFloatTensor_newWithSize3d, 4: L.THFloatTensor_newWithSize4d}[a.ndim]
        t = ctor(*a.shape)
        C.memmove(L.THFloatTensor_data(t), a.ctypes.data, a.nbytes)
        return t

    def numpy(self, t):
        """Copy of a CONTIGUOUS THFloatTensor as a numpy array."""
        L = self.lib
        shape = tuple(L.THFloatTensor_size(t, d) for d in range(L.THFloatTensor_nDimension(t)))
        out = np.empty(shape, np.float32)
        C.memmove(out.ctypes.data, L.THFloatTensor_data(t), out.nbytes)
        return out

    def free(self, *ts):
        for t in ts:
            self.lib.THFloatTensor_free(t)

    class Rng:
        def __init__(self, ref, seed):
            self._r = ref
            self._g = ref.lib.THGenerator_new()
            ref.lib.THRandom_manualSeed(self._g, seed)

        def _fill(self, fn, shape, a, b):
            t = self._r.tensor(np.empty(shape, np.float32))
            fn(t, self._g, a, b)
            out = self._r.numpy(t)
            self._r.free(t)
            return out

        def uniform(self, shape, a, b):
            return self._fill(self._r.lib.THFloatTensor_uniform, shape, a, b)

        def normal(self, shape, mean=0.0, std=1.0):
            return self._fill(self._r.lib.THFloatTensor_normal, shape, mean, std)

    def rng(self, seed):
        return _Ref.Rng(self, seed)

    # ---- fake-Lua module call ----
    def call(self, name, nums, tensors, input=None, grad_output=None, scale=None):
        """Run one ``nn`` kernel: ``nums`` / ``tensors`` are the module-table fields."""
        L = self.lib
        S = L.oref_state_new()
        keep = []
        try:
            for k, v in nums.items():
                kb = k.encode(); keep.append(kb)
                L.oref_set_num(S, kb, float(v))
            for k, v in tensors.items():
                kb = k.encode(); keep.append(kb)
                L.oref_set_ud(S, kb, v)
            if input is not None:
                L.oref_set_arg_ud(S, 2, input)
            if grad_output is not None:
                L.oref_set_arg_ud(S, 3, grad_output)
            if scale is not None:
                L.oref_set_arg_num(S, 4, scale)
            rc = L.oref_call(S, name.encode())
            if rc == -1:
                raise RuntimeError(L.oref_errmsg(S).decode())
            if rc != 0:
                raise KeyError(name)
        finally:
            L.oref_state_free(S)

    # ---- nn, through the reference's own Lua-facing functions ----
    def conv_forward(self, x, w, b, kH, kW, dH, dW, pad):
        """SpatialConvolutionMM_updateOutput; the reference raises for dW/dH != 1."""
        tx, tw, tb = self.tensor(x), self.tensor(w), self.tensor(b)
        fin, out = self.tensor(), self.tensor()
        try:
            self.call("SpatialConvolutionMM_updateOutput",
                      dict(kW=kW, kH=kH, dW=dW, dH=dH, padding=pad),
                      dict(finput=fin, weight=tw, bias=tb, output=out), input=tx)
            return self.numpy(out)
        finally:
            self.free(tx, tw, tb, fin, out)

    def conv_backward(self, x, w, go, gw, gb, scale, kH, kW, dH, dW, pad):
        """updateOutput (fills finput) + updateGradInput + accGradParameters, as Module:backward.

        Returns (gradInput, gradWeight, gradBias); gw/gb are the starting accumulators."""
        K = w.shape[0]
        tx, tw, tb = self.tensor(x), self.tensor(w), self.tensor(np.zeros(K, np.float32))
        tgo, tgw, tgb = self.tensor(go), self.tensor(gw), self.tensor(gb)
        fin, fgi, out, gi = self.tensor(), self.tensor(), self.tensor(), self.tensor()
        nums = dict(kW=kW, kH=kH, dW=dW, dH=dH, padding=pad, nOutputPlane=K)
        ts = dict(finput=fin, fgradInput=fgi, weight=tw, bias=tb, output=out, gradInput=gi,
                  gradWeight=tgw, gradBias=tgb)
        try:
            self.call("SpatialConvolutionMM_updateOutput", nums, ts, input=tx)
            # The reference multiplies the freshly resized fgradInput by beta = 0; make that defined.
            self.lib.THFloatTensor_resizeAs(fgi, fin)
            self.lib.THFloatTensor_zero(fgi)
            self.call("SpatialConvolutionMM_updateGradInput", nums, ts, input=tx, grad_output=tgo)
            self.call("SpatialConvolutionMM_accGradParameters", nums, ts, input=tx, grad_output=tgo,
                      scale=scale)
            return self.numpy(gi), self.numpy(tgw), self.numpy(tgb)
        finally:
            self.free(tx, tw, tb, tgo, tgw, tgb, fin, fgi, out, gi)

    class ConvMM:
        """A live nn.SpatialConvolutionMM on the reference's CPU code: keeps `finput` between forward
        and backward exactly as the Lua module does.  Stride 1 only (the reference's own limit)."""

        def __init__(self, ref, w, b, k, pad):
            self.r = ref
            K = w.shape[0]
            self.tw, self.tb = ref.tensor(w), ref.tensor(b)
            self.tgw, self.tgb = ref.tensor(np.zeros_like(w)), ref.tensor(np.zeros_like(b))
            self.fin, self.fgi, self.out, self.gi = ref.tensor(), ref.tensor(), ref.tensor(), ref.tensor()
            self.nums = dict(kW=k, kH=k, dW=1, dH=1, padding=pad, nOutputPlane=K)
            self.ts = dict(finput=self.fin, fgradInput=self.fgi, weight=self.tw, bias=self.tb, output=self.out,
                           gradInput=self.gi, gradWeight=self.tgw, gradBias=self.tgb)

        def forward(self, x):
            tx = self.r.tensor(x)
            try:
                self.r.call("SpatialConvolutionMM_updateOutput", self.nums, self.ts, input=tx)
                return self.r.numpy(self.out)
            finally:
                self.r.free(tx)

        def backward(self, x, go, scale=1.0, need_grad_input=True):
            tx, tgo = self.r.tensor(x), self.r.tensor(go)
            try:
                gi = None
                if need_grad_input:
                    self.r.lib.THFloatTensor_resizeAs(self.fgi, self.fin)
                    self.r.lib.THFloatTensor_zero(self.fgi)
                    self.r.call("SpatialConvolutionMM_updateGradInput", self.nums, self.ts, input=tx, grad_output=tgo)
                    gi = self.r.numpy(self.gi)
                self.r.call("SpatialConvolutionMM_accGradParameters", self.nums, self.ts, input=tx, grad_output=tgo,
                            scale=scale)
                return gi
            finally:
                self.r.free(tx, tgo)

        def grads(self):
            return self.r.numpy(self.tgw), self.r.numpy(self.tgb)

        def close(self):
            self.r.free(self.tw, self.tb, self.tgw, self.tgb, self.fin, self.fgi, self.out, self.gi)

    def conv_strided(self, x, w4, b, go, gw4, gb, scale, dH, dW, pad):
        """Stride-capable route: nn.SpatialConvolution (conv2Dmm / conv2DRevgerm) on a host-padded
        input; w4/gw4 are [K,C,kH,kW].  Returns (out, gradInput cropped, gradWeight, gradBias)."""
        K = w4.shape[0]
        xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad))) if pad else x
        full_shape = xp.shape
        # Rows/columns past the last window are never read by the forward pass; conv2DRevgerm would
        # otherwise infer a larger kernel from them, so hand the reference only the covered extent.
        kH, kW = w4.shape[2:]
        uH = (xp.shape[2] - kH) // dH * dH + kH
        uW = (xp.shape[3] - kW) // dW * dW + kW
        xp = np.ascontiguousarray(xp[:, :, :uH, :uW])
        tx, tw, tb = self.tensor(xp), self.tensor(w4), self.tensor(b)
        out, gi = self.tensor(), self.tensor()
        nums = dict(dW=dW, dH=dH, nOutputPlane=K)
        ts = dict(weight=tw, bias=tb, output=out, gradInput=gi)
        res = []
        try:
            self.call("SpatialConvolution_updateOutput", nums, ts, input=tx)
            res.append(self.numpy(out))
            if go is not None:
                tgo, tgw, tgb = self.tensor(go), self.tensor(gw4), self.tensor(gb)
                ts.update(gradWeight=tgw, gradBias=tgb)
                self.call("SpatialConvolution_updateGradInput", nums, ts, input=tx, grad_output=tgo)
                self.call("SpatialConvolution_accGradParameters", nums, ts, input=tx, grad_output=tgo,
                          scale=scale)
                g = self.numpy(gi)
                H, W = x.shape[-2:]
                # uncovered rows/columns of the padded image get zero gradient
                full = np.zeros(full_shape, np.float32)
                full[:, :, :g.shape[2], :g.shape[3]] = g
                res += [full[:, :, pad:pad + H, pad:pad + W].copy(), self.numpy(tgw), self.numpy(tgb)]
                self.free(tgo, tgw, tgb)
            return tuple(res)
        finally:
            self.free(tx, tw, tb, out, gi)

    def maxpool_forward(self, x, kH, kW, dH, dW):
        tx, out, ind = self.tensor(x), self.tensor(), self.tensor()
        try:
            self.call("SpatialMaxPooling_updateOutput", dict(kW=kW, kH=kH, dW=dW, dH=dH),
                      dict(indices=ind, output=out), input=tx)
            L = self.lib
            # indices is 5-D in batch mode; read it raw.
            nd = L.THFloatTensor_nDimension(ind)
            shape = tuple(L.THFloatTensor_size(ind, d) for d in range(nd))
            a = np.empty(shape, np.float32)
            C.memmove(a.ctypes.data, L.THFloatTensor_data(ind), a.nbytes)
            return self.numpy(out), a
        finally:
            self.free(tx, out, ind)

    def maxpool_backward(self, x, go, ind, dH, dW):
        L = self.lib
        tx, tgo, gi = self.tensor(x), self.tensor(go), self.tensor()
        tind = self.tensor(ind.reshape(2, -1, *ind.shape[-2:]))  # 4-D holder with the same memory order
        try:
            self.call("SpatialMaxPooling_updateGradInput", dict(dW=dW, dH=dH),
                      dict(indices=tind, gradInput=gi), input=tx, grad_output=tgo)
            return self.numpy(gi)
        finally:
            self.free(tx, tgo, gi, tind)

    def threshold_forward(self, x, th=0.0, val=0.0):
        tx, out = self.tensor(x), self.tensor()
        try:
            self.call("Threshold_updateOutput", dict(threshold=th, val=val), dict(output=out), input=tx)
            return self.numpy(out)
        finally:
            self.free(tx, out)

    def threshold_backward(self, x, go, th=0.0):
        tx, tgo, gi = self.tensor(x), self.tensor(go), self.tensor()
        try:
            self.call("Threshold_updateGradInput", dict(threshold=th), dict(gradInput=gi), input=tx,
                      grad_output=tgo)
            return self.numpy(gi)
        finally:
            self.free(tx, tgo, gi)

    def logsoftmax_forward(self, x):
        tx, out = self.tensor(x), self.tensor()
        try:
            self.call("LogSoftMax_updateOutput", {}, dict(output=out), input=tx)
            return self.numpy(out)
        finally:
            self.free(tx, out)

    def logsoftmax_backward(self, go, out_np):
        tgo, out, gi = self.tensor(go), self.tensor(out_np), self.tensor()
        try:
            self.call("LogSoftMax_updateGradInput", {}, dict(output=out, gradInput=gi), input=tgo,
                      grad_output=tgo)
            return self.numpy(gi)
        finally:
            self.free(tgo, out, gi)

    # ---- TH tensor math (transposed=True applies the op to t():  views, not copies) ----
    def _view(self, a):
        """THFloatTensor viewing logical array ``a``; a transposed numpy view becomes a TH transpose."""
        if a.flags["C_CONTIGUOUS"]:
            return self.tensor(a)
        assert a.ndim == 2 and a.T.flags["C_CONTIGUOUS"]
        base = self.tensor(a.T)
        v = self.lib.THFloatTensor_newTranspose(base, 0, 1)
        self.free(base)
        return v

    def add(self, t, value):
        tt, r = self._view(t), self.tensor()
        self.lib.THFloatTensor_add(r, tt, value)
        out = self.numpy(r); self.free(tt, r); return out

    def cadd(self, t, value, s):
        tt, ts, r = self._view(t), self._view(s), self.tensor()
        self.lib.THFloatTensor_cadd(r, tt, value, ts)
        out = self.numpy(r); self.free(tt, ts, r); return out

    def cmul(self, t, s):
        tt, ts, r = self._view(t), self._view(s), self.tensor()
        self.lib.THFloatTensor_cmul(r, tt, ts)
        out = self.numpy(r); self.free(tt, ts, r); return out

    def pointwise(self, name, a, b=None, c=None, v1=0.0, v2=0.0):
        """The reference's own THFloatTensor_<name> on copies of the arrays."""
        L = self.lib
        ta, r = self.tensor(a), self.tensor()
        tb = self.tensor(b) if b is not None else None
        tc = self.tensor(c) if c is not None else None
        if name in ORC_POINTWISE_NAMES[:18]:
            getattr(L, "THFloatTensor_" + name)(r, ta)
        elif name == "pow":
            L.THFloatTensor_pow(r, ta, v1)
        elif name == "clamp":
            L.THFloatTensor_clamp(r, ta, v1, v2)
        elif name == "atan2":
            L.THFloatTensor_atan2(r, ta, tb)
        elif name.endswith("Value"):
            getattr(L, "THFloatTensor_" + name + "T")(r, ta, v1)
        elif name.endswith("Tensor"):
            getattr(L, "THFloatTensor_" + name + "T")(r, ta, tb)
        else:
            getattr(L, "THFloatTensor_" + name)(r, ta, v1, tb, tc)
        out = self.numpy(r)
        self.free(*[t for t in (ta, tb, tc, r) if t is not None])
        return out

    def normall(self, t, value):
        tt = self.tensor(t); v = self.lib.THFloatTensor_normall(tt, value); self.free(tt); return v

    def dist(self, a, b, value):
        ta, tb = self.tensor(a), self.tensor(b)
        v = self.lib.THFloatTensor_dist(ta, tb, value); self.free(ta, tb); return v

    def varall(self, t):
        tt = self.tensor(t); v = self.lib.THFloatTensor_varall(tt); self.free(tt); return v

    def norm_dim(self, t, value, dim):
        tt, r = self.tensor(t), self.tensor()
        self.lib.THFloatTensor_norm(r, tt, value, dim)
        out = self.numpy(r).reshape(-1); self.free(tt, r); return out

    def _long(self, idx):
        L = self.lib
        idx = np.ascontiguousarray(idx, np.int64)
        t = L.THLongTensor_newWithSize1d(idx.size)
        C.memmove(L.THLongTensor_data(t), idx.ctypes.data, idx.nbytes)
        return t

    def prodall(self, t):
        tt = self.tensor(t); v = self.lib.THFloatTensor_prodall(tt); self.free(tt); return v

    def prod_dim(self, t, dim):
        tt, r = self.tensor(t), self.tensor()
        self.lib.THFloatTensor_prod(r, tt, dim)
        out = self.numpy(r); self.free(tt, r); return out

    def renorm(self, t, value, dim, maxnorm):
        tt, r = self.tensor(t), self.tensor()
        self.lib.THFloatTensor_renorm(r, tt, value, dim, maxnorm)
        out = self.numpy(r); self.free(tt, r); return out

    def index_select(self, t, dim, idx):
        tt, r, ti = self.tensor(t), self.tensor(), self._long(idx)
        self.lib.THFloatTensor_indexSelect(r, tt, dim, ti)
        out = self.numpy(r); self.free(tt, r); self.lib.THLongTensor_free(ti); return out

    def index_copy(self, res, dim, idx, src):
        tr, ts, ti = self.tensor(res), self.tensor(src), self._long(idx)
        self.lib.THFloatTensor_indexCopy(tr, dim, ti, ts)
        out = self.numpy(tr); self.free(tr, ts); self.lib.THLongTensor_free(ti); return out

    def index_fill(self, res, dim, idx, val):
        tr, ti = self.tensor(res), self._long(idx)
        self.lib.THFloatTensor_indexFill(tr, dim, ti, val)
        out = self.numpy(tr); self.free(tr); self.lib.THLongTensor_free(ti); return out

    def softmax_forward(self, x):
        tx, out = self.tensor(x), self.tensor()
        try:
            self.call("SoftMax_updateOutput", {}, dict(output=out), input=tx)
            return self.numpy(out)
        finally:
            self.free(tx, out)

    def softmax_backward(self, go, out_np):
        tgo, out, gi = self.tensor(go), self.tensor(out_np), self.tensor()
        try:
            self.call("SoftMax_updateGradInput", {}, dict(output=out, gradInput=gi), input=tgo, grad_output=tgo)
            return self.numpy(gi)
        finally:
            self.free(tgo, out, gi)

    def sumpool_forward(self, x, kH, kW, dH, dW):
        tx, out = self.tensor(x), self.tensor()
        try:
            self.call("SpatialAveragePooling_updateOutput", dict(kW=kW, kH=kH, dW=dW, dH=dH), dict(output=out), input=tx)
            return self.numpy(out)
        finally:
            self.free(tx, out)

    def sumpool_backward(self, x, go, kH, kW, dH, dW):
        tx, tgo, gi = self.tensor(x), self.tensor(go), self.tensor()
        try:
            self.call("SpatialAveragePooling_updateGradInput", dict(kW=kW, kH=kH, dW=dW, dH=dH), dict(gradInput=gi),
                      input=tx, grad_output=tgo)
            return self.numpy(gi)
        finally:
            self.free(tx, tgo, gi)

    def sumall(self, t):
        tt = self._view(t); v = self.lib.THFloatTensor_sumall(tt); self.free(tt); return v

    def maxall(self, t):
        tt = self._view(t); v = self.lib.THFloatTensor_maxall(tt); self.free(tt); return v

    def sum_dim(self, t, dim):
        tt, r = self._view(t), self.tensor()
        self.lib.THFloatTensor_sum(r, tt, dim)
        out = self.numpy(r).reshape(-1); self.free(tt, r); return out

    def max_dim(self, t, dim):
        L = self.lib
        tt, r, idx = self._view(t), self.tensor(), L.THLongTensor_new()
        L.THFloatTensor_max(r, idx, tt, dim)
        out = self.numpy(r).reshape(-1)
        n = out.size
        ia = np.empty(n, np.int64)
        C.memmove(ia.ctypes.data, L.THLongTensor_data(idx), ia.nbytes)
        self.free(tt, r); L.THLongTensor_free(idx)
        return out, ia

    def addmm(self, beta, t, alpha, m1, m2):
        tt, a, b = self.tensor(t), self._view(m1), self._view(m2)
        self.lib.THFloatTensor_addmm(tt, beta, tt, alpha, a, b)
        out = self.numpy(tt); self.free(tt, a, b); return out


ref = _Ref()

"""`torch.GPUTensor` for Python hosts: a thin object over the THGPUTensor C ABI.

Method names, argument order and overloads follow the Lua methods the reference registers for
`torch.GPUTensor` (gputorch/TensorMath.cpp:6076-6229 method table; gputorch/Tensor.lua:7-40 for the
`:gpu()` / `:float()` conversions).  Dimension arguments are 1-based, as in Lua.  Host tensors
(`torch.FloatTensor` in the reference) are numpy float32 arrays here.  All arithmetic happens in
the CUDA library; nothing in this file computes on the CPU."""
import ctypes as C

import numpy as np

from ._lib import (THFloatStorage, THFloatTensor, THLongStorage, lib)


def _long_storage(values):
    arr = (C.c_long * len(values))(*values)
    s = THLongStorage()
    s.data = C.cast(arr, C.POINTER(C.c_long))
    s.size = len(values)
    s.refcount = 1
    s._keep = arr
    return s


def _host_view(a):
    """THFloatTensor struct describing numpy array ``a`` in place (any strides, float32)."""
    assert isinstance(a, np.ndarray) and a.dtype == np.float32
    if a.ndim == 0:
        a = a.reshape(1)
    for st in a.strides:
        assert st % 4 == 0 and st >= 0, "unsupported numpy strides"
    st = THFloatStorage()
    st.data = C.cast(C.c_void_p(a.ctypes.data), C.POINTER(C.c_float))
    st.size = 1 + sum((n - 1) * (s // 4) for n, s in zip(a.shape, a.strides)) if a.size else 0
    st.refcount = 1
    t = THFloatTensor()
    size = (C.c_long * a.ndim)(*a.shape)
    stride = (C.c_long * a.ndim)(*[s // 4 for s in a.strides])
    t.size = C.cast(size, C.POINTER(C.c_long))
    t.stride = C.cast(stride, C.POINTER(C.c_long))
    t.nDimension = a.ndim if a.size else 0
    t.storage = C.pointer(st)
    t.storageOffset = 0
    t.refcount = 1
    t._keep = (a, st, size, stride)
    return t


class GPUTensor:
    """torch.GPUTensor.  Construct empty, with sizes, or from a numpy float32 array (copies)."""

    __slots__ = ("_p",)

    def __init__(self, *args, _ptr=None):
        L = lib()
        if _ptr is not None:
            self._p = _ptr
            return
        if len(args) == 1 and isinstance(args[0], np.ndarray):
            a = np.asarray(args[0], dtype=np.float32)
            self._p = L.THGPUTensor_new()
            if a.size:
                self.resize(*a.shape)
                self.copy(a)
            return
        self._p = L.THGPUTensor_new()
        if args:
            self.resize(*args)

    def __del__(self):
        try:
            if self._p:
                lib().cdll.THGPUTensor_free(self._p)
        except Exception:
            pass

    # ---- metadata (host only) ----
    @property
    def cdata(self):
        return self._p

    def dim(self):
        return self._p.contents.nDimension

    nDimension = dim

    def size(self, d=None):
        t = self._p.contents
        if d is None:
            return tuple(t.size[k] for k in range(t.nDimension))
        return lib().THGPUTensor_size(self._p, d - 1)

    def stride(self, d=None):
        t = self._p.contents
        if d is None:
            return tuple(t.stride[k] for k in range(t.nDimension))
        return lib().THGPUTensor_stride(self._p, d - 1)

    def storageOffset(self):
        return self._p.contents.storageOffset + 1

    def nElement(self):
        return lib().THGPUTensor_nElement(self._p)

    def isContiguous(self):
        return bool(lib().THGPUTensor_isContiguous(self._p))

    def data_ptr(self):
        return lib().THGPUTensor_data(self._p) or 0

    def type(self):
        return "torch.GPUTensor"

    # ---- shape ----
    def resize(self, *sizes):
        if len(sizes) == 1 and isinstance(sizes[0], (tuple, list)):
            sizes = tuple(sizes[0])
        s = _long_storage([int(v) for v in sizes])
        lib().THGPUTensor_resize(self._p, C.byref(s), None)
        return self

    def resizeAs(self, other):
        lib().THGPUTensor_resizeAs(self._p, other._p)
        return self

    def set(self, other):
        lib().THGPUTensor_set(self._p, other._p)
        return self

    def t(self):
        assert self.dim() == 2
        return GPUTensor(_ptr=lib().THGPUTensor_newTranspose(self._p, 0, 1))

    def transpose(self, d1, d2):
        return GPUTensor(_ptr=lib().THGPUTensor_newTranspose(self._p, d1 - 1, d2 - 1))

    def narrow(self, d, first, size):
        return GPUTensor(_ptr=lib().THGPUTensor_newNarrow(self._p, d - 1, first - 1, size))

    def select(self, d, index):
        return GPUTensor(_ptr=lib().THGPUTensor_newSelect(self._p, d - 1, index - 1))

    def view(self, *sizes):
        assert self.isContiguous(), "view needs a contiguous tensor"
        n = self.nElement()
        sizes = list(sizes)
        if -1 in sizes:
            k = sizes.index(-1)
            rest = int(np.prod([s for s in sizes if s != -1])) or 1
            sizes[k] = n // rest
        assert int(np.prod(sizes)) == n
        L = lib()
        r = GPUTensor()
        s = _long_storage(sizes)
        L.THGPUTensor_setStorage(r._p, self._p.contents.storage, self._p.contents.storageOffset, C.byref(s), None)
        return r

    def contiguous(self):
        return GPUTensor(_ptr=lib().THGPUTensor_newContiguous(self._p))

    def clone(self):
        return GPUTensor(_ptr=lib().THGPUTensor_newClone(self._p))

    # ---- copies / conversions ----
    def copy(self, src):
        L = lib()
        if isinstance(src, GPUTensor):
            L.THGPUTensor_copy(self._p, src._p)
        else:
            a = np.asarray(src, dtype=np.float32)
            h = _host_view(a)
            L.THGPUTensor_copyFloat(self._p, C.byref(h))
        return self

    def float(self, out=None):
        """Device -> host: numpy float32 array of this tensor's shape (`:float()`)."""
        shape = self.size() if self.dim() else (0,)
        if out is None:
            out = np.empty(shape, np.float32)
        if out.size:
            h = _host_view(out)
            lib().THFloatTensor_copyGPU(C.byref(h), self._p)
        return out

    def gpu(self):
        return self

    # ---- fill ----
    def fill(self, v):
        lib().THGPUTensor_fill(self._p, float(v))
        return self

    def zero(self):
        lib().THGPUTensor_zero(self._p)
        return self

    # ---- elementwise: x:add(v) | x:add(y) | x:add(v, y) | x:add(a, v) | x:add(a, y) | x:add(a, v, b) ----
    def add(self, *a):
        L = lib()
        if len(a) == 1 and not isinstance(a[0], GPUTensor):
            L.THGPUTensor_add(self._p, self._p, float(a[0]))
        elif len(a) == 1:
            L.THGPUTensor_cadd(self._p, self._p, 1.0, a[0]._p)
        elif len(a) == 2 and not isinstance(a[0], GPUTensor):
            L.THGPUTensor_cadd(self._p, self._p, float(a[0]), a[1]._p)
        elif len(a) == 2 and not isinstance(a[1], GPUTensor):
            L.THGPUTensor_add(self._p, a[0]._p, float(a[1]))
        elif len(a) == 2:
            L.THGPUTensor_cadd(self._p, a[0]._p, 1.0, a[1]._p)
        elif len(a) == 3:
            L.THGPUTensor_cadd(self._p, a[0]._p, float(a[1]), a[2]._p)
        else:
            raise TypeError("add: bad arguments")
        return self

    def mul(self, *a):
        if len(a) == 1:
            lib().THGPUTensor_mul(self._p, self._p, float(a[0]))
        else:
            lib().THGPUTensor_mul(self._p, a[0]._p, float(a[1]))
        return self

    def div(self, *a):
        if len(a) == 1:
            lib().THGPUTensor_div(self._p, self._p, float(a[0]))
        else:
            lib().THGPUTensor_div(self._p, a[0]._p, float(a[1]))
        return self

    def cmul(self, *a):
        if len(a) == 1:
            lib().THGPUTensor_cmul(self._p, self._p, a[0]._p)
        else:
            lib().THGPUTensor_cmul(self._p, a[0]._p, a[1]._p)
        return self

    def cdiv(self, *a):
        if len(a) == 1:
            lib().THGPUTensor_cdiv(self._p, self._p, a[0]._p)
        else:
            lib().THGPUTensor_cdiv(self._p, a[0]._p, a[1]._p)
        return self

    # pointwise functions: t:log() works in place, r:log(t) writes log(t) into r (the cwrap'd Lua overloads,
    # gputorch/TensorMath.cpp:6076-6229)
    def _unary(self, name, a):
        src = a[0] if a else self
        getattr(lib(), "THGPUTensor_" + name)(self._p, src._p)
        return self

    def pow(self, *a):
        if len(a) == 1:
            lib().THGPUTensor_pow(self._p, self._p, float(a[0]))
        else:
            lib().THGPUTensor_pow(self._p, a[0]._p, float(a[1]))
        return self

    def clamp(self, *a):
        if len(a) == 2:
            lib().THGPUTensor_clamp(self._p, self._p, float(a[0]), float(a[1]))
        else:
            lib().THGPUTensor_clamp(self._p, a[0]._p, float(a[1]), float(a[2]))
        return self

    def atan2(self, tx, ty):
        lib().THGPUTensor_atan2(self._p, tx._p, ty._p)
        return self

    def _compare(self, name, a):
        # r:lt(t, value) / r:lt(t1, t2); t:lt(value) and t:lt(t2) return a new tensor of 1.0 / 0.0
        if len(a) == 1:
            out, src, rhs = GPUTensor(), self, a[0]
        else:
            out, src, rhs = self, a[0], a[1]
        if isinstance(rhs, GPUTensor):
            getattr(lib(), "THGPUTensor_%sTensor" % name)(out._p, src._p, rhs._p)
        else:
            getattr(lib(), "THGPUTensor_%sValue" % name)(out._p, src._p, float(rhs))
        return out

    def addcmul(self, *a):
        """t:addcmul(value, src1, src2) in place, r:addcmul(t, value, src1, src2) into r."""
        t, value, s1, s2 = (self,) + a if len(a) == 3 else a
        lib().THGPUTensor_addcmul(self._p, t._p, float(value), s1._p, s2._p)
        return self

    def addcdiv(self, *a):
        t, value, s1, s2 = (self,) + a if len(a) == 3 else a
        lib().THGPUTensor_addcdiv(self._p, t._p, float(value), s1._p, s2._p)
        return self

    def norm(self, *a):
        """t:norm([value]) -> number; r:norm(t, value, dim) -> r (dim 1-based, like the Lua method)."""
        if len(a) == 3:
            lib().THGPUTensor_norm(self._p, a[0]._p, float(a[1]), int(a[2]) - 1)
            return self
        return lib().THGPUTensor_normall(self._p, float(a[0]) if a else 2.0)

    def dist(self, other, value=2.0):
        return lib().THGPUTensor_dist(self._p, other._p, float(value))

    def var(self):
        return lib().THGPUTensor_varall(self._p)

    def std(self):
        return lib().THGPUTensor_stdall(self._p)

    def dot(self, other):
        return lib().THGPUTensor_dot(self._p, other._p)

    # ---- reductions: x:sum() -> number; x:sum(dim) -> tensor; r:sum(x, dim) ----
    def _reduce(self, allfn, dimfn, a, with_indices):
        L = lib()
        if len(a) == 0:
            return allfn(self._p)
        if len(a) == 1:
            src, dim = self, a[0]
            val = GPUTensor()
            if with_indices:
                idx = GPUTensor()
                dimfn(val._p, idx._p, src._p, dim - 1)
                return val, idx
            dimfn(val._p, src._p, dim - 1)
            return val
        src, dim = a
        if with_indices:
            idx = GPUTensor()
            dimfn(self._p, idx._p, src._p, dim - 1)
            return self, idx
        dimfn(self._p, src._p, dim - 1)
        return self

    def sum(self, *a):
        return self._reduce(lib().THGPUTensor_sumall, lib().THGPUTensor_sum, a, False)

    def mean(self, *a):
        return self._reduce(lib().THGPUTensor_meanall, lib().THGPUTensor_mean, a, False)

    def max(self, *a):
        return self._reduce(lib().THGPUTensor_maxall, lib().THGPUTensor_max, a, True)

    def min(self, *a):
        return self._reduce(lib().THGPUTensor_minall, lib().THGPUTensor_min, a, True)

    # ---- products: r:addmm([beta,] [t,] [alpha,] m1, m2) as the cwrap overloads resolve them ----
    @staticmethod
    def _blas_args(self_t, a, n_tensors):
        nums = [x for x in a if not isinstance(x, GPUTensor)]
        tens = [x for x in a if isinstance(x, GPUTensor)]
        lead = []
        for x in a:
            if isinstance(x, GPUTensor):
                break
            lead.append(x)
        if len(tens) == n_tensors + 1:
            t = tens[0]
            tens = tens[1:]
        else:
            t = self_t
        if len(nums) == 0:
            beta, alpha = 1.0, 1.0
        elif len(nums) == 1:
            beta, alpha = 1.0, float(nums[0])
        else:
            beta, alpha = float(nums[0]), float(nums[1])
        return beta, t, alpha, tens

    def addmm(self, *a):
        beta, t, alpha, (m1, m2) = self._blas_args(self, a, 2)
        lib().THGPUTensor_addmm(self._p, beta, t._p, alpha, m1._p, m2._p)
        return self

    def addmv(self, *a):
        beta, t, alpha, (m, v) = self._blas_args(self, a, 2)
        lib().THGPUTensor_addmv(self._p, beta, t._p, alpha, m._p, v._p)
        return self

    def addr(self, *a):
        beta, t, alpha, (v1, v2) = self._blas_args(self, a, 2)
        lib().THGPUTensor_addr(self._p, beta, t._p, alpha, v1._p, v2._p)
        return self

    def mm(self, m1, m2):
        self.resize(m1.size(1), m2.size(2))
        lib().THGPUTensor_addmm(self._p, 0.0, self._p, 1.0, m1._p, m2._p)
        return self

    def __repr__(self):
        return "torch.GPUTensor of size %s" % "x".join(str(s) for s in self.size())


def gpu(a):
    """`:gpu()` for a host tensor: numpy array -> new GPUTensor (gputorch/Tensor.lua:7-25)."""
    if isinstance(a, GPUTensor):
        return a
    return GPUTensor(np.ascontiguousarray(a, dtype=np.float32))


def synchronize():
    lib().THGPUSynchronize()


def set_device(dev):
    """gputorch.setDevice (1-based, like Lua)."""
    lib().THGPUSetDevice(dev - 1)


def get_device_count():
    return lib().THGPUGetDeviceCount()


MATH_MODES = {"fp32x3": 0, "simt": 1, "bf16": 2}


def set_math_mode(name):
    lib().THGPUBlas_setMathMode(MATH_MODES[name])


def _install_pointwise_methods():
    from ._lib import COMPARISONS, UNARY_FUNCTIONS
    for name in UNARY_FUNCTIONS:
        setattr(GPUTensor, name, (lambda n: lambda self, *a: self._unary(n, a))(name))
    for name in COMPARISONS:
        setattr(GPUTensor, name, (lambda n: lambda self, *a: self._compare(n, a))(name))


_install_pointwise_methods()

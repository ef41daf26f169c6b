"""`torch.GPUTensor` for Python hosts: a thin object over the THGPUTensor C ABI.

Method names, argument order and overloads follow the Lua methods the reference registers for
`torch.GPUTensor` (gputorch/TensorMath.cpp:6076-6229 method table; gputorch/Tensor.lua:7-40 for the
`:gpu()` / `:float()` conversions).  Dimension arguments are 1-based, as in Lua.  Host tensors
(`torch.FloatTensor` in the reference) are numpy float32 arrays here.  All arithmetic happens in
the CUDA library; nothing in this file computes on the CPU."""
import ctypes as C

import numpy as np

from ._lib import (HOST_TYPES, THLongStorage, lib)

# numpy dtype -> TH host type name
_TH_NAME = {np.dtype(v[0]): k for k, v in HOST_TYPES.items()}


def _long_storage(values):
    arr = (C.c_long * len(values))(*values)
    s = THLongStorage()
    s.data = C.cast(arr, C.POINTER(C.c_long))
    s.size = len(values)
    s.refcount = 1
    s._keep = arr
    return s


def _host_view(a):
    """(TH type name, TH<Type>Tensor struct) describing numpy array ``a`` in place (any strides; one of the
    seven TH element types)."""
    assert isinstance(a, np.ndarray) and a.dtype in _TH_NAME, "no TH host tensor type for dtype %s" % a.dtype
    name = _TH_NAME[a.dtype]
    _, storage_t, tensor_t = HOST_TYPES[name]
    if a.ndim == 0:
        a = a.reshape(1)
    isz = a.dtype.itemsize
    for st in a.strides:
        assert st % isz == 0 and st >= 0, "unsupported numpy strides"
    st = storage_t()
    st.data = C.cast(C.c_void_p(a.ctypes.data), type(st.data))
    st.size = 1 + sum((n - 1) * (s // isz) for n, s in zip(a.shape, a.strides)) if a.size else 0
    st.refcount = 1
    t = tensor_t()
    size = (C.c_long * a.ndim)(*a.shape)
    stride = (C.c_long * a.ndim)(*[s // isz for s in a.strides])
    t.size = C.cast(size, C.POINTER(C.c_long))
    t.stride = C.cast(stride, C.POINTER(C.c_long))
    t.nDimension = a.ndim if a.size else 0
    t.storage = C.pointer(st)
    t.storageOffset = 0
    t.refcount = 1
    t._keep = (a, st, size, stride)
    return name, t


class GPUTensor:
    """torch.GPUTensor.  Construct empty, with sizes, or from a numpy float32 array (copies)."""

    __slots__ = ("_p",)

    def __init__(self, *args, _ptr=None):
        L = lib()
        if _ptr is not None:
            self._p = _ptr
            return
        if len(args) == 1 and isinstance(args[0], np.ndarray):
            a = args[0] if args[0].dtype in _TH_NAME else np.asarray(args[0], dtype=np.float32)
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
            # a host tensor of any TH type: THGPUTensor_copy<Type> (gputorch/Tensor.cpp:38-65 dispatches the same way)
            a = np.asarray(src)
            if a.dtype not in _TH_NAME:
                a = a.astype(np.float32)
            name, h = _host_view(a)
            getattr(L, "THGPUTensor_copy" + name)(self._p, C.byref(h))
        return self

    def _to_host(self, dtype, out):
        shape = self.size() if self.dim() else (0,)
        if out is None:
            out = np.empty(shape, dtype)
        if out.size:
            name, h = _host_view(out)
            getattr(lib(), "TH%sTensor_copyGPU" % name)(C.byref(h), self._p)
        return out

    def float(self, out=None):
        """Device -> host: numpy float32 array of this tensor's shape (`:float()`)."""
        return self._to_host(np.float32, out)

    def double(self, out=None):
        """`:double()` (gputorch/Tensor.lua:26-28): host float64 array."""
        return self._to_host(np.float64, out)

    def long(self, out=None):
        return self._to_host(np.int64, out)

    def int(self, out=None):
        return self._to_host(np.int32, out)

    def short(self, out=None):
        return self._to_host(np.int16, out)

    def char(self, out=None):
        return self._to_host(np.int8, out)

    def byte(self, out=None):
        return self._to_host(np.uint8, out)

    def gpu(self):
        return self

    # ---- object serialisation: pickle / copy.deepcopy see a tensor as (storage object, header record), the
    # two pieces the reference's Tensor write / read handle (gputorch/torch/generic/Tensor.c:1150-1199); the
    # storage object is shared by every tensor that views it, so a flattened parameter storage is written once
    # and the views still share it after loading, as with Lua's file:writeObject ----
    def storage(self):
        sp = self._p.contents.storage
        return GPUStorage._of(sp) if sp else None

    def __reduce__(self):
        import io
        from ._lib import file_callbacks
        buf = io.BytesIO()
        f = file_callbacks(buf)
        lib().THGPUTensor_writeHeader(self._p, C.byref(f))
        return (_tensor_from_parts, (self.storage(), buf.getvalue()))

    # ---- serialisation (torch.save / torch.load records of a GPU tensor) ----
    def write(self, fh):
        """Writes this tensor's record (header, storage) to the binary file object `fh`."""
        from ._lib import file_callbacks
        f = file_callbacks(fh)
        lib().THGPUTensor_write(self._p, C.byref(f))
        return self

    def read(self, fh):
        """Replaces this tensor by the record read from `fh` (fresh storage)."""
        from ._lib import file_callbacks
        f = file_callbacks(fh)
        lib().THGPUTensor_read(self._p, C.byref(f))
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

    # ---- x:renorm(p, dim, maxnorm) | x:renorm(src, p, dim, maxnorm) ----
    def renorm(self, *a):
        src = self
        if isinstance(a[0], GPUTensor):
            src, a = a[0], a[1:]
        p, dim, maxnorm = a
        lib().THGPUTensor_renorm(self._p, src._p, float(p), dim - 1, float(maxnorm))
        return self

    # ---- index operations: `index` is a host LongTensor (any integer sequence) of 1-based positions ----
    @staticmethod
    def _index(index):
        return _host_view(np.ascontiguousarray(index, dtype=np.int64).reshape(-1))[1]

    def index(self, dim, index):
        """x:index(dim, idx): new tensor of the selected slices"""
        r = GPUTensor()
        lib().THGPUTensor_indexSelect(r._p, self._p, dim - 1, C.byref(self._index(index)))
        return r

    def indexSelect(self, src, dim, index):
        lib().THGPUTensor_indexSelect(self._p, src._p, dim - 1, C.byref(self._index(index)))
        return self

    def indexCopy(self, dim, index, src):
        lib().THGPUTensor_indexCopy(self._p, dim - 1, C.byref(self._index(index)), src._p)
        return self

    def indexFill(self, dim, index, val):
        lib().THGPUTensor_indexFill(self._p, dim - 1, C.byref(self._index(index)), float(val))
        return self

    # ---- x:zeros(sizes) | x:ones(sizes) | x:reshape(src, sizes) ----
    def zeros(self, *sizes):
        lib().THGPUTensor_zeros(self._p, C.byref(_long_storage(list(sizes))))
        return self

    def ones(self, *sizes):
        lib().THGPUTensor_ones(self._p, C.byref(_long_storage(list(sizes))))
        return self

    def reshape(self, *a):
        src = self
        if isinstance(a[0], GPUTensor):
            src, a = a[0], a[1:]
        lib().THGPUTensor_reshape(self._p, src._p, C.byref(_long_storage(list(a))))
        return self

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

    def prod(self, *a):
        return self._reduce(lib().THGPUTensor_prodall, lib().THGPUTensor_prod, a, False)

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


class GPUStorage:
    """torch.GPUStorage: one Python object per THGPUStorage while any reference to it lives."""

    _live = None

    def __init__(self, _ptr):
        self._p = _ptr          # retained by _of / _storage_from_bytes

    @classmethod
    def _of(cls, sp):
        import weakref
        if cls._live is None:
            cls._live = weakref.WeakValueDictionary()
        key = C.addressof(sp.contents)
        obj = cls._live.get(key)
        if obj is None:
            lib().THGPUStorage_retain(sp)
            obj = cls(sp)
            cls._live[key] = obj
        return obj

    def __del__(self):
        try:
            if self._p:
                lib().cdll.THGPUStorage_free(self._p)
        except Exception:
            pass

    def size(self):
        return lib().THGPUStorage_size(self._p)

    def __reduce__(self):
        import io
        from ._lib import file_callbacks
        buf = io.BytesIO()
        f = file_callbacks(buf)
        lib().THGPUStorage_write(self._p, C.byref(f))
        return (_storage_from_bytes, (buf.getvalue(),))


def _storage_from_bytes(record):
    import io
    from ._lib import file_callbacks
    L = lib()
    sp = L.THGPUStorage_new()
    f = file_callbacks(io.BytesIO(record))
    try:
        L.THGPUStorage_read(sp, C.byref(f))
    except Exception:
        L.THGPUStorage_free(sp)
        raise
    obj = GPUStorage(sp)        # owns the reference THGPUStorage_new returned
    if GPUStorage._live is None:
        import weakref
        GPUStorage._live = weakref.WeakValueDictionary()
    GPUStorage._live[C.addressof(sp.contents)] = obj
    return obj


def _tensor_from_parts(storage, header):
    import io
    from ._lib import file_callbacks
    t = GPUTensor()
    f = file_callbacks(io.BytesIO(header))
    lib().THGPUTensor_readHeader(t._p, storage._p if storage is not None else None, C.byref(f))
    return t


def save(obj, path):
    """torch.save for objects that hold GPU tensors (modules, tables of tensors): pickle, with every
    torch.GPUTensor / torch.GPUStorage written as the reference's binary records."""
    import pickle
    with open(path, "wb") as fh:
        pickle.dump(obj, fh, protocol=4)


def load(path):
    import pickle
    with open(path, "rb") as fh:
        return pickle.load(fh)


def gpu(a):
    """`:gpu()` for a host tensor: numpy array -> new GPUTensor (gputorch/Tensor.lua:7-25)."""
    if isinstance(a, GPUTensor):
        return a
    a = np.asarray(a)
    # any of the seven TH host types converts on the device (Torch7's default tensor type is Double)
    return GPUTensor(a if a.dtype in _TH_NAME else np.ascontiguousarray(a, dtype=np.float32))


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

"""ctypes binding of libTHC.so: the same stub a LuaJIT FFI / luaT wrapper would write.

The library must have been built (``python -m mcw_cppamp_torch_b200.build``); there is no fallback:
if it is missing, or no CUDA device is present, calls fail loudly."""
import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libTHC.so")


class THLongStorage(C.Structure):
    _fields_ = [("data", C.POINTER(C.c_long)), ("size", C.c_long), ("refcount", C.c_int), ("flag", C.c_char),
                ("allocator", C.c_void_p), ("allocatorContext", C.c_void_p)]


class THFloatStorage(C.Structure):
    _fields_ = [("data", C.POINTER(C.c_float)), ("size", C.c_long), ("refcount", C.c_int), ("flag", C.c_char),
                ("allocator", C.c_void_p), ("allocatorContext", C.c_void_p)]


class THFloatTensor(C.Structure):
    _fields_ = [("size", C.POINTER(C.c_long)), ("stride", C.POINTER(C.c_long)), ("nDimension", C.c_int),
                ("storage", C.POINTER(THFloatStorage)), ("storageOffset", C.c_long), ("refcount", C.c_int),
                ("flag", C.c_char)]


def _host_types(name, ctype, st=None):
    """TH<name>Storage / TH<name>Tensor: the layout of THFloatStorage / THFloatTensor with another element type."""
    st = st or type("TH%sStorage" % name, (C.Structure,), {"_fields_": [
        ("data", C.POINTER(ctype)), ("size", C.c_long), ("refcount", C.c_int), ("flag", C.c_char),
        ("allocator", C.c_void_p), ("allocatorContext", C.c_void_p)]})
    tn = type("TH%sTensor" % name, (C.Structure,), {"_fields_": [
        ("size", C.POINTER(C.c_long)), ("stride", C.POINTER(C.c_long)), ("nDimension", C.c_int),
        ("storage", C.POINTER(st)), ("storageOffset", C.c_long), ("refcount", C.c_int), ("flag", C.c_char)]})
    return st, tn


# host element types by TH name: (numpy dtype name, storage struct, tensor struct)
HOST_TYPES = {"Float": ("float32", THFloatStorage, THFloatTensor)}
for _name, _ct, _np in (("Byte", C.c_ubyte, "uint8"), ("Char", C.c_byte, "int8"), ("Short", C.c_short, "int16"),
                        ("Int", C.c_int, "int32"), ("Double", C.c_double, "float64")):
    HOST_TYPES[_name] = (_np,) + _host_types(_name, _ct)
HOST_TYPES["Long"] = ("int64",) + _host_types("Long", C.c_long, THLongStorage)


class THGPUStorage(C.Structure):
    _fields_ = [("data", C.POINTER(C.c_float)), ("size", C.c_long), ("refcount", C.c_int), ("flag", C.c_char),
                ("allocator", C.c_void_p), ("allocatorContext", C.c_void_p)]


class THGPUTensor(C.Structure):
    _fields_ = [("size", C.POINTER(C.c_long)), ("stride", C.POINTER(C.c_long)), ("nDimension", C.c_int),
                ("storage", C.POINTER(THGPUStorage)), ("storageOffset", C.c_long), ("refcount", C.c_int),
                ("flag", C.c_char)]


_FILE_WRITE = C.CFUNCTYPE(C.c_long, C.c_void_p, C.c_void_p, C.c_long)
_FILE_READ = C.CFUNCTYPE(C.c_long, C.c_void_p, C.c_void_p, C.c_long)


class THGPUFile(C.Structure):
    _fields_ = [("write", _FILE_WRITE), ("read", _FILE_READ), ("ctx", C.c_void_p)]


def file_callbacks(fh):
    """THGPUFile over a Python binary file object (anything with write(bytes) / read(n))."""
    def _w(ctx, data, n):
        try:
            return fh.write(C.string_at(data, n)) if n else 0
        except Exception:
            return -1

    def _r(ctx, data, n):
        try:
            b = fh.read(n) if n else b""
            C.memmove(data, b, len(b))
            return len(b)
        except Exception:
            return -1
    f = THGPUFile(_FILE_WRITE(_w), _FILE_READ(_r), None)
    f._keep = (_w, _r, fh)
    return f


class THGPUCommBackend(C.Structure):
    """Transport callbacks of a THGPUComm (include/THC.h)."""
    ALL_REDUCE = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_long, C.c_long)
    SET_UPDATE = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float)
    DONE = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int)
    JOIN = C.CFUNCTYPE(C.c_int, C.c_void_p)
    AGREE = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_long), C.c_int)
    ABORT = C.CFUNCTYPE(C.c_int, C.c_void_p)
    DESTROY = C.CFUNCTYPE(None, C.c_void_p)
    _fields_ = [("all_reduce", ALL_REDUCE), ("set_update", SET_UPDATE), ("done", DONE), ("join", JOIN),
                ("agree", AGREE), ("abort", ABORT), ("destroy", DESTROY), ("ctx", C.c_void_p)]


TP = C.POINTER(THGPUTensor)
SP = C.POINTER(THGPUStorage)
LSP = C.POINTER(THLongStorage)
FTP = C.POINTER(THFloatTensor)
FSP = C.POINTER(THFloatStorage)
f, l, i, d, vp, ch = C.c_float, C.c_long, C.c_int, C.c_double, C.c_void_p, C.c_char
fp = C.POINTER(C.c_float)

# name -> (restype, argtypes); every symbol include/THC.h declares
SIGNATURES = {
    "THGPUInit": (None, []), "THGPUShutdown": (None, []), "THGPUGetDeviceCount": (i, []),
    "THGPUSetDevice": (None, [i]), "THGPUGetDevice": (i, []), "THGPUSynchronize": (None, []),
    "THGPUGetStream": (vp, []), "THGPUSetStream": (None, [vp]), "THGPUGetLastError": (C.c_char_p, []),
    "THGPUClearError": (None, []), "THGPUSetErrorHandler": (None, [vp, vp]),
    "THGPUBlas_setMathMode": (None, [i]), "THGPUBlas_getMathMode": (i, []), "THGPUKernelLaunchCount": (l, []),
    "THGPUSetWaitLimit": (None, [l]), "THGPUGetWaitLimit": (l, []), "THGPUStallProbe": (i, [l]),
    "THGPUDeviceAllocCount": (l, []),
    "THGPUStorage_data": (fp, [SP]), "THGPUStorage_size": (l, [SP]), "THGPUStorage_set": (None, [SP, l, f]),
    "THGPUStorage_get": (f, [SP, l]), "THGPUStorage_new": (SP, []), "THGPUStorage_newWithSize": (SP, [l]),
    "THGPUStorage_newWithData": (SP, [vp, l]), "THGPUStorage_retain": (None, [SP]), "THGPUStorage_free": (None, [SP]),
    "THGPUStorage_fill": (None, [SP, f]), "THGPUStorage_resize": (None, [SP, l]), "THGPUStorage_rawCopy": (None, [SP, vp]),
    "THGPUStorage_copy": (None, [SP, SP]), "THGPUStorage_copyGPU": (None, [SP, SP]),
    "THGPUTensor_storage": (SP, [TP]), "THGPUTensor_storageOffset": (l, [TP]), "THGPUTensor_nDimension": (i, [TP]),
    "THGPUTensor_size": (l, [TP, i]), "THGPUTensor_stride": (l, [TP, i]), "THGPUTensor_data": (vp, [TP]),
    "THGPUTensor_new": (TP, []), "THGPUTensor_newWithTensor": (TP, [TP]),
    "THGPUTensor_newWithStorage": (TP, [SP, l, LSP, LSP]), "THGPUTensor_newWithStorage1d": (TP, [SP, l, l, l]),
    "THGPUTensor_newWithStorage2d": (TP, [SP, l, l, l, l, l]), "THGPUTensor_newWithSize": (TP, [LSP, LSP]),
    "THGPUTensor_newWithSize1d": (TP, [l]), "THGPUTensor_newWithSize2d": (TP, [l, l]),
    "THGPUTensor_newWithSize3d": (TP, [l, l, l]), "THGPUTensor_newWithSize4d": (TP, [l, l, l, l]),
    "THGPUTensor_newClone": (TP, [TP]), "THGPUTensor_newContiguous": (TP, [TP]),
    "THGPUTensor_newSelect": (TP, [TP, i, l]), "THGPUTensor_newNarrow": (TP, [TP, i, l, l]),
    "THGPUTensor_newTranspose": (TP, [TP, i, i]), "THGPUTensor_resize": (None, [TP, LSP, LSP]),
    "THGPUTensor_resizeAs": (None, [TP, TP]), "THGPUTensor_resize1d": (None, [TP, l]),
    "THGPUTensor_resize2d": (None, [TP, l, l]), "THGPUTensor_resize3d": (None, [TP, l, l, l]),
    "THGPUTensor_resize4d": (None, [TP, l, l, l, l]), "THGPUTensor_resize5d": (None, [TP, l, l, l, l, l]),
    "THGPUTensor_set": (None, [TP, TP]), "THGPUTensor_setStorage": (None, [TP, SP, l, LSP, LSP]),
    "THGPUTensor_narrow": (None, [TP, TP, i, l, l]), "THGPUTensor_select": (None, [TP, TP, i, l]),
    "THGPUTensor_transpose": (None, [TP, TP, i, i]), "THGPUTensor_squeeze": (None, [TP, TP]),
    "THGPUTensor_isContiguous": (i, [TP]), "THGPUTensor_isSameSizeAs": (i, [TP, TP]), "THGPUTensor_nElement": (l, [TP]),
    "THGPUTensor_retain": (None, [TP]), "THGPUTensor_free": (None, [TP]), "THGPUTensor_freeCopyTo": (None, [TP, TP]),
    "THGPUTensor_set1d": (None, [TP, l, f]), "THGPUTensor_set2d": (None, [TP, l, l, f]),
    "THGPUTensor_get1d": (f, [TP, l]), "THGPUTensor_get2d": (f, [TP, l, l]),
    "THGPUTensor_copy": (None, [TP, TP]), "THGPUTensor_copyGPU": (None, [TP, TP]),
    "THGPUStorage_write": (i, [SP, C.POINTER(THGPUFile)]), "THGPUStorage_read": (i, [SP, C.POINTER(THGPUFile)]),
    "THGPUTensor_writeHeader": (i, [TP, C.POINTER(THGPUFile)]),
    "THGPUTensor_readHeader": (i, [TP, SP, C.POINTER(THGPUFile)]),
    "THGPUTensor_write": (i, [TP, C.POINTER(THGPUFile)]), "THGPUTensor_read": (i, [TP, C.POINTER(THGPUFile)]),
    "THGPUComm_getUniqueId": (i, [vp]), "THGPUComm_new": (vp, [i, i, vp]),
    "THGPUComm_newWithOptions": (vp, [i, i, vp, i]),
    "THGPUComm_newWithBackend": (vp, [i, i, C.POINTER(THGPUCommBackend)]), "THGPUComm_free": (None, [vp]),
    "THGPUComm_setTimeout": (i, [vp, d]), "THGPUComm_setBuckets": (i, [vp, TP, C.POINTER(C.c_long), i]),
    "THGPUComm_setUpdate": (i, [vp, TP, TP, f, f]), "THGPUComm_allReduceAsync": (i, [vp, i]),
    "THGPUComm_wait": (i, [vp]), "THGPUComm_error": (C.c_char_p, [vp]),
    "THGPUTensor_fill": (None, [TP, f]), "THGPUTensor_zero": (None, [TP]), "THGPUTensor_numel": (l, [TP]),
    "THGPUTensor_add": (None, [TP, TP, f]), "THGPUTensor_mul": (None, [TP, TP, f]), "THGPUTensor_div": (None, [TP, TP, f]),
    "THGPUTensor_cadd": (None, [TP, TP, f, TP]), "THGPUTensor_cmul": (None, [TP, TP, TP]),
    "THGPUTensor_cdiv": (None, [TP, TP, TP]), "THGPUTensor_dot": (f, [TP, TP]), "THGPUTensor_minall": (f, [TP]),
    "THGPUTensor_maxall": (f, [TP]), "THGPUTensor_sumall": (f, [TP]), "THGPUTensor_meanall": (f, [TP]),
    "THGPUTensor_sumall_noalloc": (i, [vp, l, vp, vp]),
    "THGPUTensor_min": (None, [TP, TP, TP, l]), "THGPUTensor_max": (None, [TP, TP, TP, l]),
    "THGPUTensor_sum": (None, [TP, TP, l]), "THGPUTensor_mean": (None, [TP, TP, l]),
    "THGPUTensor_addmv": (None, [TP, f, TP, f, TP, TP]), "THGPUTensor_addmm": (None, [TP, f, TP, f, TP, TP]),
    "THGPUTensor_addr": (None, [TP, f, TP, f, TP, TP]),
    "THGPUTensor_addcmul": (None, [TP, TP, f, TP, TP]), "THGPUTensor_addcdiv": (None, [TP, TP, f, TP, TP]),
    "THGPUTensor_pow": (None, [TP, TP, f]), "THGPUTensor_clamp": (None, [TP, TP, f, f]),
    "THGPUTensor_atan2": (None, [TP, TP, TP]),
    "THGPUTensor_varall": (f, [TP]), "THGPUTensor_stdall": (f, [TP]), "THGPUTensor_normall": (f, [TP, f]),
    "THGPUTensor_dist": (f, [TP, TP, f]),
    "THGPUTensor_norm": (None, [TP, TP, f, l]),
    "THGPUTensor_zeros": (None, [TP, LSP]), "THGPUTensor_ones": (None, [TP, LSP]),
    "THGPUTensor_reshape": (None, [TP, TP, LSP]), "THGPUTensor_prodall": (f, [TP]),
    "THGPUTensor_prod": (None, [TP, TP, l]), "THGPUTensor_renorm": (None, [TP, TP, f, l, f]),
    "THGPUTensor_indexCopy": (None, [TP, i, C.POINTER(HOST_TYPES["Long"][2]), TP]),
    "THGPUTensor_indexFill": (None, [TP, i, C.POINTER(HOST_TYPES["Long"][2]), f]),
    "THGPUTensor_indexSelect": (None, [TP, TP, i, C.POINTER(HOST_TYPES["Long"][2])]),
    "THGPUNN_SoftMax_updateOutput": (i, [TP, TP]), "THGPUNN_SoftMax_updateGradInput": (i, [TP, TP, TP, TP]),
    "THGPUNN_SpatialAveragePooling_updateOutput": (i, [TP, TP, i, i, i, i]),
    "THGPUNN_SpatialAveragePooling_updateGradInput": (i, [TP, TP, TP, i, i, i, i]),
    "THGPUBlas_gemm": (None, [ch, ch, l, l, l, f, vp, l, vp, l, f, vp, l]),
    "THGPUBlas_gemv": (None, [ch, l, l, f, vp, l, vp, l, f, vp, l]),
    "THGPUBlas_axpy": (None, [l, f, vp, l, vp, l]), "THGPUBlas_ger": (None, [l, l, f, vp, l, vp, l, vp, l]),
    "THGPUNN_SpatialConvolutionMM_updateOutput": (i, [TP, TP, TP, TP, TP, TP, i, i, i, i, i]),
    "THGPUNN_SpatialConvolutionMM_updateGradInput": (i, [TP, TP, TP, TP, TP, TP, i, i, i, i, i]),
    "THGPUNN_SpatialConvolutionMM_accGradParameters": (i, [TP, TP, TP, TP, TP, TP, i, i, i, i, i, f]),
    "THGPUNN_SpatialConvolutionMM_backward": (i, [TP, TP, TP, TP, TP, TP, TP, TP, i, i, i, i, i, f]),
    "THGPUNN_SpatialMaxPooling_updateOutput": (i, [TP, TP, TP, i, i, i, i]),
    "THGPUNN_SpatialMaxPooling_updateGradInput": (i, [TP, TP, TP, TP, i, i, i, i]),
    "THGPUNN_Threshold_updateOutput": (i, [TP, TP, d, d]), "THGPUNN_Threshold_updateGradInput": (i, [TP, TP, TP, d]),
    "THGPUNN_LogSoftMax_updateOutput": (i, [TP, TP]), "THGPUNN_LogSoftMax_updateGradInput": (i, [TP, TP, TP, TP]),
    "THGPUNN_ClassNLLCriterion_updateOutput": (i, [TP, TP, TP, i]),
    "THGPUNN_ClassNLLCriterion_updateGradInput": (i, [TP, TP, TP, i]),
    "THGPUNN_SGD_update": (i, [TP, TP, TP, f, f]),
}

for _n, (_np, _st, _tn) in HOST_TYPES.items():
    SIGNATURES["THGPUStorage_copy" + _n] = (None, [SP, C.POINTER(_st)])
    SIGNATURES["TH%sStorage_copyGPU" % _n] = (None, [C.POINTER(_st), SP])
    SIGNATURES["THGPUTensor_copy" + _n] = (None, [TP, C.POINTER(_tn)])
    SIGNATURES["TH%sTensor_copyGPU" % _n] = (None, [C.POINTER(_tn), TP])

UNARY_FUNCTIONS = ("log", "log1p", "exp", "cos", "acos", "cosh", "sin", "asin", "sinh", "tan", "atan", "tanh",
                   "sqrt", "ceil", "floor", "abs", "sign", "round")
COMPARISONS = ("lt", "gt", "le", "ge", "eq", "ne")
for _n in UNARY_FUNCTIONS:
    SIGNATURES["THGPUTensor_" + _n] = (None, [TP, TP])
for _n in COMPARISONS:
    SIGNATURES["THGPUTensor_%sValue" % _n] = (None, [TP, TP, f])
    SIGNATURES["THGPUTensor_%sTensor" % _n] = (None, [TP, TP, TP])


class THCError(RuntimeError):
    """What a Lua wrapper would raise through THError / luaL_error."""


class _Lib:
    def __init__(self):
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: build it with `python -m mcw_cppamp_torch_b200.build` "
                              "(there is no CPU fallback)" % LIB_PATH)
        self.cdll = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(self.cdll, name)
            fn.restype = res
            fn.argtypes = args
            if name not in ("THGPUGetLastError", "THGPUClearError"):
                setattr(self, name, self._checked(fn))
            else:
                setattr(self, name, fn)

    def _checked(self, fn):
        get, clear = self.cdll.THGPUGetLastError, self.cdll.THGPUClearError

        def call(*a):
            r = fn(*a)
            e = get()
            if e is not None:
                msg = e.decode()
                clear()
                raise THCError(msg)
            return r
        call.raw = fn
        return call


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = _Lib()
    return _lib

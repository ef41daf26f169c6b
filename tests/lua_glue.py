"""Builds the library's Lua glue against the fake Lua of tests/lua_shim and wraps the driver for the tests."""
import ctypes as C
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SHIM = os.path.join(HERE, "lua_shim")
OUT = os.path.join(SHIM, "_build", "libgluetest.so")
GPU = b"torch.GPUTensor"


def build():
    import __graft_entry__
    __graft_entry__.build()
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    srcs = [os.path.join(ROOT, "mcw_cppamp_torch_b200", "lua", "gpunn_glue.c"),
            os.path.join(ROOT, "mcw_cppamp_torch_b200", "lua", "gputorch_glue.c"), os.path.join(SHIM, "fake_lua.c")]
    pkg = os.path.join(ROOT, "mcw_cppamp_torch_b200")
    subprocess.check_call(["gcc", "-std=gnu99", "-O1", "-Wall", "-Werror", "-shared", "-fPIC", "-I", SHIM,
                           "-I", os.path.join(ROOT, "include")] + srcs +
                          ["-L", pkg, "-lTHC", "-Wl,-rpath," + pkg, "-o", OUT])
    return OUT


class FakeLua:
    """One fake lua_State with both libraries' registration done on demand."""

    def __init__(self):
        from mcw_cppamp_torch_b200 import lib
        lib()                                     # libTHC.so is in the process before the glue asks for it
        L = C.CDLL(build())
        vp = C.c_void_p
        L.fl_new.restype = vp
        L.fl_free.argtypes = [vp]
        L.fl_errmsg.argtypes = [vp]; L.fl_errmsg.restype = C.c_char_p
        L.fl_clear_call.argtypes = [vp]
        L.fl_arg_ud.argtypes = [vp, C.c_int, vp, C.c_char_p]
        L.fl_arg_num.argtypes = [vp, C.c_int, C.c_double]
        L.fl_field_num.argtypes = [vp, C.c_char_p, C.c_double]
        L.fl_field_bool.argtypes = [vp, C.c_char_p, C.c_int]
        L.fl_field_ud.argtypes = [vp, C.c_char_p, vp, C.c_char_p]
        L.fl_open.argtypes = [vp, C.c_int]
        L.fl_registered.argtypes = [vp]
        L.fl_registered_owner.argtypes = [vp, C.c_int]; L.fl_registered_owner.restype = C.c_char_p
        L.fl_registered_name.argtypes = [vp, C.c_int]; L.fl_registered_name.restype = C.c_char_p
        L.fl_call.argtypes = [vp, C.c_char_p, C.c_char_p]
        L.fl_result.argtypes = [vp, C.c_int]; L.fl_result.restype = C.c_double
        self.L, self.S = L, L.fl_new()
        self._keep = []

    def open(self, which):
        rc = self.L.fl_open(self.S, {"gpunn": 0, "gputorch": 1}[which])
        if rc < 0:
            raise RuntimeError(self.L.fl_errmsg(self.S).decode())
        return rc

    def registered(self):
        return [(self.L.fl_registered_owner(self.S, i).decode(), self.L.fl_registered_name(self.S, i).decode())
                for i in range(self.L.fl_registered(self.S))]

    def call(self, owner, name, args=(), fields=None):
        """args: slot 2, 3, ... values (a (pointer, type name) pair, a number, or None); slot 1 is the module table,
        whose fields are `fields` (numbers, bools, or (pointer, type name) pairs).  Returns (number of Lua results,
        [pushed numbers]); raises RuntimeError with the Lua error message."""
        L, S = self.L, self.S
        L.fl_clear_call(S)
        self._keep = []

        def ptr(p):
            return C.cast(p, C.c_void_p)
        first = 1 if fields is None else 2
        for k, a in enumerate(args):
            if a is None:
                continue
            if isinstance(a, tuple):
                L.fl_arg_ud(S, first + k, ptr(a[0]), a[1])
            else:
                L.fl_arg_num(S, first + k, float(a))
        for key, v in (fields or {}).items():
            kb = key.encode(); self._keep.append(kb)
            if isinstance(v, tuple):
                L.fl_field_ud(S, kb, ptr(v[0]), v[1])
            elif isinstance(v, bool):
                L.fl_field_bool(S, kb, int(v))
            else:
                L.fl_field_num(S, kb, float(v))
        rc = L.fl_call(S, owner.encode(), name.encode())
        if rc == -1:
            raise RuntimeError(L.fl_errmsg(S).decode())
        if rc == -2:
            raise KeyError((owner, name))
        return rc, [L.fl_result(S, i) for i in range(4)]

    def module_fields(self, m):
        """The Lua module table of a Python mirror module: every number / bool / GPUTensor attribute, by its name."""
        from mcw_cppamp_torch_b200 import GPUTensor
        out = {}
        for k, v in m.__dict__.items():
            if isinstance(v, GPUTensor):
                out[k] = (v._p, GPU)
            elif isinstance(v, (bool, int, float)):
                out[k] = v
        return out

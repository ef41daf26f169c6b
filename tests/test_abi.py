"""CPU-only checks of the drop-in boundary: the built library exports every symbol include/THC.h
declares, the Python binding covers them all, and host-side tensor metadata behaves like TH."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    src = open(os.path.join(ROOT, "include", "THC.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"THC_API\s+[\w\s\*]+?\b(\w+)\s*\(", src)))


@pytest.fixture(scope="module")
def cdll():
    import __graft_entry__
    __graft_entry__.build()
    from mcw_cppamp_torch_b200._lib import LIB_PATH
    return C.CDLL(LIB_PATH)


def test_every_declared_symbol_is_exported(cdll):
    names = _declared()
    assert len(names) > 100
    missing = [n for n in names if not hasattr(cdll, n)]
    assert not missing, missing


def test_binding_covers_the_header():
    from mcw_cppamp_torch_b200._lib import SIGNATURES
    assert sorted(SIGNATURES) == _declared()


def test_struct_layouts_match_the_ffi_declaration():
    # gputorch/FFI.lua:5-29: {float*, long, int, char, ptr, ptr} and {long*, long*, int, ptr, long, int, char}
    from mcw_cppamp_torch_b200._lib import THGPUStorage, THGPUTensor
    assert [f[0] for f in THGPUStorage._fields_] == ["data", "size", "refcount", "flag", "allocator", "allocatorContext"]
    assert [f[0] for f in THGPUTensor._fields_] == ["size", "stride", "nDimension", "storage", "storageOffset", "refcount", "flag"]
    assert C.sizeof(THGPUStorage) == 40 and C.sizeof(THGPUTensor) == 48
    assert THGPUTensor.storageOffset.offset == 32 and THGPUStorage.allocatorContext.offset == 32


def test_views_and_contiguity_on_borrowed_storage():
    """Metadata-only operations need no device: use a storage that borrows a (never dereferenced) pointer."""
    from mcw_cppamp_torch_b200 import lib
    L = lib()
    st = L.THGPUStorage_newWithData(C.c_void_p(0x1000), 2 * 3 * 4)
    t = L.THGPUTensor_newWithStorage2d(st, 0, 6, 4, 4, 1)
    assert L.THGPUTensor_isContiguous(t) == 1 and L.THGPUTensor_nElement(t) == 24
    tt = L.THGPUTensor_newTranspose(t, 0, 1)
    assert L.THGPUTensor_isContiguous(tt) == 0
    assert (L.THGPUTensor_size(tt, 0), L.THGPUTensor_stride(tt, 0)) == (4, 1)
    nr = L.THGPUTensor_newNarrow(t, 0, 2, 3)
    assert L.THGPUTensor_storageOffset(nr) == 8 and L.THGPUTensor_size(nr, 0) == 3
    assert L.THGPUTensor_isContiguous(nr) == 1
    nc = L.THGPUTensor_newNarrow(t, 1, 1, 2)
    assert L.THGPUTensor_isContiguous(nc) == 0
    sel = L.THGPUTensor_newSelect(t, 1, 3)
    assert L.THGPUTensor_nDimension(sel) == 1 and L.THGPUTensor_stride(sel, 0) == 4
    assert L.THGPUTensor_storageOffset(sel) == 3
    # size-1 dims are ignored by isContiguous (gputorch/lib/THC/THCTensor.cpp:510-525)
    one = L.THGPUTensor_newNarrow(tt, 1, 1, 1)  # sizes (4,1), strides (1,4)
    assert L.THGPUTensor_isContiguous(one) == 1
    # storage refcount: 1 (ours) + five tensors
    assert st.contents.refcount == 7
    for x in (t, tt, nr, nc, sel, one):
        L.THGPUTensor_free(x)
    assert st.contents.refcount == 1
    L.THGPUStorage_free(st)


def test_errors_are_reported_not_fatal():
    from mcw_cppamp_torch_b200 import lib, THCError
    L = lib()
    st = L.THGPUStorage_newWithData(C.c_void_p(0x1000), 8)
    t = L.THGPUTensor_newWithStorage1d(st, 0, 8, 1)
    with pytest.raises(THCError, match="out of range"):
        L.THGPUTensor_newNarrow(t, 0, 4, 9)
    with pytest.raises(THCError, match="not resizable"):
        L.THGPUStorage_resize(st, 100)
    assert L.THGPUGetLastError() is None  # cleared after being raised
    L.THGPUTensor_free(t)
    L.THGPUStorage_free(st)


def test_compute_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from mcw_cppamp_torch_b200 import GPUTensor, THCError
    with pytest.raises(THCError, match="no CUDA device"):
        GPUTensor(4)


def test_header_compiles_as_c_and_cxx_and_a_c_program_links(tmp_path):
    """The boundary is a C ABI: include/THC.h must be valid C99 and C++ on its own, and a plain C program that
    includes it links against the library and calls an entry point that needs no device."""
    import shutil
    import subprocess
    root = os.path.join(os.path.dirname(__file__), "..")
    inc = os.path.join(root, "include")
    libdir = os.path.join(root, "mcw_cppamp_torch_b200")
    if not shutil.which("gcc") or not shutil.which("g++"):
        pytest.skip("no host compiler")
    src = tmp_path / "use_thc.c"
    src.write_text('#include "THC.h"\n#include <stdio.h>\n'
                   'int main(void) {\n'
                   '  THGPUClearError();\n'
                   '  const char *e = THGPUGetLastError();\n'
                   '  printf("%s %d\\n", e ? e : "none", (int)sizeof(THGPUTensor));\n'
                   '  return e ? 1 : 0;\n}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-I", inc, str(src)], check=True)
    subprocess.run(["g++", "-std=c++17", "-Wall", "-fsyntax-only", "-x", "c++", "-I", inc, str(src)], check=True)
    exe = tmp_path / "use_thc"
    subprocess.run(["gcc", "-std=c99", "-I", inc, str(src), "-o", str(exe), "-L", libdir, "-l:libTHC.so",
                    "-Wl,-rpath," + os.path.abspath(libdir)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert out[0] == "none" and int(out[1]) > 0

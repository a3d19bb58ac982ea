"""TEST INFRASTRUCTURE: Python face of oracle/x86_regalloc.cpp, the restatement of the reference's
register-allocating x86-64 CPU back end (crates/basalt-x86/src/regalloc.rs).  A compiled kernel is
called the way the reference's C drivers call theirs (examples/cpu_launch_*.c): the kernel's own
parameters followed by `int64 nthreads`; the body runs once per thread, one thread at a time.

    k = compile(bir_text)
    k(a_ptr, b_ptr, c_ptr, n, nthreads)
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libx86regalloc.so")

_lib = None


class Refused(Exception):
    """check_module said no: `code` is the reference's E-code (E090 op, E091 type, E093 feature)."""

    def __init__(self, code: str, arg: str):
        super().__init__(f"{code}: {arg}")
        self.code = code
        self.arg = arg


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            from . import build
            build.build()
        l = C.CDLL(LIB)
        l.orx_compile.argtypes = [C.c_char_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p, C.c_char_p, C.c_size_t]
        l.orx_compile.restype = C.c_int
        l.orx_entry.argtypes = [C.c_void_p]
        l.orx_entry.restype = C.c_void_p
        l.orx_code.argtypes = [C.c_void_p, C.POINTER(C.POINTER(C.c_uint8))]
        l.orx_code.restype = C.c_size_t
        l.orx_signature.argtypes = [C.c_void_p]
        l.orx_signature.restype = C.c_char_p
        l.orx_name.argtypes = [C.c_void_p]
        l.orx_name.restype = C.c_char_p
        l.orx_spills.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
        l.orx_spills.restype = None
        l.orx_free.argtypes = [C.c_void_p]
        l.orx_free.restype = None
        _lib = l
    return _lib


_CTYPES = {"i1": C.c_uint8, "i8": C.c_int8, "i16": C.c_int16, "i32": C.c_int32, "i64": C.c_int64, "f32": C.c_float, "f64": C.c_double,
           "void": None}


def _ctype(ty: str):
    return C.c_void_p if ty.startswith("ptr.") else _CTYPES[ty]


class Kernel:
    def __init__(self, handle):
        self._h = handle
        l = lib()
        params, ret = l.orx_signature(handle).decode().split("->")
        self.params = params.split()
        self.ret = ret.strip()
        self.name = l.orx_name(handle).decode()
        proto = C.CFUNCTYPE(_ctype(self.ret), *[_ctype(p) for p in self.params], C.c_int64)
        self._fn = proto(l.orx_entry(handle))
        ints, floats = C.c_uint32(), C.c_uint32()
        l.orx_spills(handle, C.byref(ints), C.byref(floats))
        self.int_spills, self.float_spills = ints.value, floats.value

    @property
    def code(self) -> bytes:
        p = C.POINTER(C.c_uint8)()
        n = lib().orx_code(self._h, C.byref(p))
        return C.string_at(p, n)

    def __call__(self, *args):
        """args = the kernel's parameters then nthreads.  numpy arrays are passed by address."""
        if len(args) != len(self.params) + 1:
            raise TypeError(f"{self.name} takes {len(self.params)} parameters and nthreads")
        conv = [a.ctypes.data if hasattr(a, "ctypes") else a for a in args]
        return self._fn(*conv)

    def __del__(self):
        try:
            lib().orx_free(self._h)
        except Exception:
            pass


def compile(bir: str) -> Kernel:
    src = bir.encode()
    out, code, msg = C.c_void_p(), C.create_string_buffer(8), C.create_string_buffer(512)
    rc = lib().orx_compile(src, len(src), C.byref(out), code, msg, len(msg))
    if rc == 1:
        raise Refused(code.value.decode(), msg.value.decode())
    if rc != 0:
        raise OSError(msg.value.decode())
    return Kernel(out)

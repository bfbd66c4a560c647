"""ctypes binding of the eddl_b200 C ABI (``include/eddl_b200.h``).

Argument types are derived from the header itself, so the binding cannot drift from the
declarations.  Loading fails loudly when the CUDA library has not been built: there is no CPU
fallback behind this module.
"""
import ctypes
import os
import re

import numpy as np

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
HEADER = os.path.join(ROOT, "include", "eddl_b200.h")
LIBPATH = os.path.join(PKG, "lib", "libeddl_b200.so")

_SCALARS = {"int": ctypes.c_int, "float": ctypes.c_float, "size_t": ctypes.c_size_t}


def declared_functions(header=HEADER):
    """[(name, restype_str, [param_type_str, ...])] for every function the header declares."""
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    out = []
    for m in re.finditer(r"(const char \*|int)\s*(eddlb200_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        ret, name, params = m.group(1).strip(), m.group(2), " ".join(m.group(3).split())
        plist = [] if params in ("void", "") else [p.strip() for p in params.split(",")]
        out.append((name, ret, plist))
    return out


def _ctype(param):
    if "*" in param:
        return ctypes.c_void_p
    base = param.replace("const", " ").split()
    return _SCALARS[base[0]] if base[0] in _SCALARS else ctypes.c_int


class Error(RuntimeError):
    pass


class Lib:
    """The loaded C ABI.  ``lib.call('conv2d_fwd', dev, ...)`` raises Error on a non-zero status."""

    def __init__(self, path=LIBPATH):
        if not os.path.exists(path):
            raise ImportError("eddl_b200: %s is missing -- build it with `python eddl_b200/build.py kernels` "
                              "(there is no CPU fallback)" % path)
        self.cdll = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
        self.fn = {}
        for name, ret, params in declared_functions():
            f = getattr(self.cdll, name)
            f.restype = ctypes.c_char_p if "char" in ret else ctypes.c_int
            f.argtypes = [_ctype(p) for p in params]
            self.fn[name[len("eddlb200_"):]] = f

    def last_error(self):
        return self.fn["last_error"]().decode()

    def call(self, name, *args):
        conv = [a.ptr if isinstance(a, DeviceArray) else a for a in args]
        st = self.fn[name](*conv)
        if st != 0:
            raise Error("eddlb200_%s -> %d: %s" % (name, st, self.last_error()))

    def device_count(self):
        n = ctypes.c_int(0)
        st = self.fn["device_count"](ctypes.byref(n))
        return n.value if st == 0 else 0

    # -- device arrays ---------------------------------------------------------------------
    def empty(self, shape, dev=0):
        return DeviceArray(self, tuple(np.atleast_1d(shape)) if not isinstance(shape, tuple) else shape, dev)

    def to_device(self, arr, dev=0):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        d = DeviceArray(self, arr.shape, dev)
        if arr.size:
            self.call("memcpy_h2d", dev, d.ptr, arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes)
        return d

    def zeros(self, shape, dev=0):
        d = self.empty(shape, dev)
        if d.size:
            self.call("fill", dev, d.ptr, d.size, 0.0)
        return d

    def sync(self, dev=0):
        self.call("sync", dev)

    def launches(self, dev=0):
        n = ctypes.c_ulonglong(0)
        self.call("launch_count", dev, ctypes.byref(n))
        return n.value


class DeviceArray:
    """fp32 device buffer owned through eddlb200_alloc / eddlb200_free."""

    def __init__(self, lib, shape, dev=0):
        self.lib, self.shape, self.dev = lib, tuple(int(s) for s in shape), dev
        self.size = int(np.prod(self.shape)) if len(self.shape) else 1
        p = ctypes.c_void_p()
        lib.call("alloc", dev, max(self.size, 1) * 4, ctypes.byref(p))
        self.ptr = p

    def numpy(self):
        out = np.empty(self.shape, dtype=np.float32)
        if self.size:
            self.lib.call("memcpy_d2h", self.dev, out.ctypes.data_as(ctypes.c_void_p), self.ptr, out.nbytes)
        return out

    def __del__(self):
        try:
            if self.ptr:
                self.lib.fn["free"](self.dev, self.ptr)
                self.ptr = None
        except Exception:
            pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = Lib()
    return _lib

"""ctypes view of the C ABI (include/greta_cuda.h, include/greta_host.h).

Signatures are generated from the headers themselves, so a declaration that the
library does not export fails at load time.  Device memory is handled through
the ABI's own allocator (`DeviceBuffer`); nothing here computes on the host.
"""
import ctypes as C
import os
import re

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
INCLUDE_DIR = os.path.join(_ROOT, "include")

FMT_F16, FMT_REF_INT8, FMT_REF_INT4, FMT_Q4_0, FMT_Q8_0 = 1, 3, 4, 8, 9
PAYLOAD_BYTES = {FMT_Q4_0: 16, FMT_Q8_0: 32}
GGUF_BLOCK_BYTES = {FMT_Q4_0: 18, FMT_Q8_0: 34}

_SCALARS = {
    "int": C.c_int, "long long": C.c_longlong, "float": C.c_float, "double": C.c_double, "uint32_t": C.c_uint32, "int32_t": C.c_int32,
    "uint64_t": C.c_uint64, "int64_t": C.c_int64, "size_t": C.c_size_t, "greta_stream_t": C.c_void_p,
    "greta_model_t": C.c_void_p,
}
_DECL = re.compile(r"GRETA_API\s+([\w\s\*]+?)\s*\b(greta_\w+)\s*\(([^;]*?)\)\s*;", re.S)


def _ctype(text):
    t = " ".join(text.replace("const", " ").split())
    if "*" in t:
        return C.c_char_p if t.replace(" ", "") == "char*" and "const" in text else C.c_void_p
    return _SCALARS[t]


def parse_header(path):
    """-> list of (name, restype, [argtypes]) for every GRETA_API declaration in the header."""
    src = re.sub(r"/\*.*?\*/", "", open(path).read(), flags=re.S)
    src = re.sub(r"//[^\n]*", "", src)
    out = []
    for ret, name, args in _DECL.findall(src):
        args = args.strip()
        argtypes = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                base = re.sub(r"\b\w+$", "", a).strip() if not a.endswith("*") else a   # drop the parameter name
                argtypes.append(_ctype(base))
        out.append((name, _ctype(ret), argtypes))
    return out


class GretaError(RuntimeError):
    pass


_libs = {}


def _load(libname, header):
    if libname in _libs:
        return _libs[libname]
    path = os.path.join(_HERE, libname)
    if not os.path.exists(path):
        raise GretaError(f"{libname} is not built: run `python -c 'import __graft_entry__ as g; g.build()'` "
                         "(there is no CPU fallback)")
    lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
    for name, restype, argtypes in parse_header(os.path.join(INCLUDE_DIR, header)):
        fn = getattr(lib, name)          # AttributeError if the header declares what the library lacks
        fn.restype, fn.argtypes = restype, argtypes
    _libs[libname] = lib
    return lib


def cuda():
    return _load("libgreta_cuda.so", "greta_cuda.h")


def host():
    cuda()
    return _load("libgreta_host.so", "greta_host.h")


def check(rc, what=""):
    if rc != 0:
        msg = cuda().greta_cuda_last_error()
        raise GretaError(f"{what or 'greta_cuda call'} failed with code {rc}: {msg.decode() if msg else ''}")


def device_count():
    n = C.c_int(0)
    rc = cuda().greta_cuda_device_count(C.byref(n))
    return n.value if rc == 0 else 0


def require_device():
    if device_count() < 1:
        raise GretaError("no CUDA device visible: this path has no CPU fallback")


class DeviceBuffer:
    """Device memory owned through greta_cuda_malloc / greta_cuda_free."""

    def __init__(self, nbytes, zero=False):
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        check(cuda().greta_cuda_malloc(C.byref(p), self.nbytes), "greta_cuda_malloc")
        self.ptr = p.value
        if zero:
            check(cuda().greta_cuda_memset(self.ptr, 0, self.nbytes, None))
            check(cuda().greta_cuda_device_synchronize())

    @classmethod
    def from_numpy(cls, arr):
        arr = np.ascontiguousarray(arr)
        buf = cls(max(arr.nbytes, 1))
        buf.upload(arr)
        return buf

    def upload(self, arr, offset=0):
        arr = np.ascontiguousarray(arr)
        assert offset + arr.nbytes <= self.nbytes
        if arr.nbytes:
            check(cuda().greta_cuda_memcpy_h2d_sync(self.ptr + offset, arr.ctypes.data, arr.nbytes), "memcpy_h2d")

    def download(self, dtype, count=None, offset=0):
        dtype = np.dtype(dtype)
        if count is None:
            count = (self.nbytes - offset) // dtype.itemsize
        out = np.empty(count, dtype)
        if out.nbytes:
            check(cuda().greta_cuda_memcpy_d2h_sync(out.ctypes.data, self.ptr + offset, out.nbytes), "memcpy_d2h")
        return out

    def fill(self, byte):
        check(cuda().greta_cuda_memset(self.ptr, byte, self.nbytes, None))
        check(cuda().greta_cuda_device_synchronize())

    def free(self):
        if getattr(self, "ptr", None):
            cuda().greta_cuda_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Weight:
    """A quantised [N x K] weight resident on the device in the planar layout."""

    def __init__(self, gguf_blocks, fmt, N, K):
        lib = cuda()
        self.fmt, self.N, self.K = fmt, N, K
        blocks = np.ascontiguousarray(gguf_blocks, np.uint8)
        assert blocks.size == N * (K // 32) * GGUF_BLOCK_BYTES[fmt]
        raw = DeviceBuffer.from_numpy(blocks)
        self.qs = DeviceBuffer(max(lib.greta_cuda_qs_bytes(fmt, N, K), 16))
        self.d = DeviceBuffer(max(lib.greta_cuda_d_bytes(fmt, N, K), 16))
        check(lib.greta_cuda_repack_gguf(None, fmt, raw.ptr, self.qs.ptr, self.d.ptr, N, K), "repack_gguf")
        check(lib.greta_cuda_device_synchronize())
        raw.free()

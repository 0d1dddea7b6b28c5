"""B200-native quantized-matmul hot path for GRETA CORE.

The product is two shared libraries built from csrc/: libgreta_cuda.so (sm_100a
kernels behind the C ABI of include/greta_cuda.h) and libgreta_host.so (the C++
host layer that mirrors the reference's gcore:: API on top of that C ABI).
This Python package only loads them through ctypes for the tests and the
benchmark; it holds no compute of its own and has no CPU fallback: if the CUDA
library is missing or no device is present, calls raise.
"""
from . import ffi, model, rendezvous  # noqa: F401
from .build import build  # noqa: F401

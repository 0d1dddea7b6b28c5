"""Shared helpers of the test-suite: package loading, seeded GGUF block makers, error metric."""
import os
import struct
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load_package():
    """The package under its importable name (the loader lives beside the build entry point)."""
    from __graft_entry__ import load_package as _load
    return _load()


def q4_0_blocks(rng, N, K, sigma=0.02):
    """GGUF Q4_0 blocks of W[N,K]: q uniform in 0..15, d = |N(0,sigma)|/8 as fp16 (the prefill-GEMM benchmark distribution)."""
    nb = N * (K // 32)
    blk = np.empty((nb, 18), np.uint8)
    blk[:, :2] = (np.abs(rng.normal(0, sigma, nb)) / 8).astype(np.float16).view(np.uint8).reshape(nb, 2)
    blk[:, 2:] = rng.integers(0, 256, (nb, 16), dtype=np.uint8)
    return blk.reshape(-1)


def q8_0_blocks(rng, N, K, sigma=0.02):
    """GGUF Q8_0 blocks: q uniform in [-127,127], d = |N(0,sigma)|/127 as fp16 (the Q8_0 GEMV benchmark distribution)."""
    nb = N * (K // 32)
    blk = np.empty((nb, 34), np.uint8)
    blk[:, :2] = (np.abs(rng.normal(0, sigma, nb)) / 127).astype(np.float16).view(np.uint8).reshape(nb, 2)
    blk[:, 2:] = rng.integers(-127, 128, (nb, 32), dtype=np.int8).view(np.uint8)
    return blk.reshape(-1)


def make_blocks(rng, fmt, N, K):
    from oracle import oracle as O
    return q4_0_blocks(rng, N, K) if fmt == O.FMT_Q4_0 else q8_0_blocks(rng, N, K)


def max_abs_rel(got, want):
    """max |got - want| / max |want|: the acceptance metric (<= 2e-3 for matmul and attention)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    denom = np.abs(want).max()
    return float(np.abs(got - want).max() / (denom if denom > 0 else 1.0))


def _s(b):
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, kv_u32, kv_f32, tensors):
    """Minimal GGUF v3 writer: u32 / f32 metadata and raw tensors (name, dims, ggml type, bytes).
    dims are given outermost-first and stored innermost-first as GGUF does."""
    out = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kv_u32) + len(kv_f32)))
    for k, v in kv_u32:
        out += _s(k.encode()) + struct.pack("<II", 4, v)
    for k, v in kv_f32:
        out += _s(k.encode()) + struct.pack("<If", 6, v)
    off = 0
    for name, dims, gtype, data in tensors:
        out += _s(name.encode()) + struct.pack("<I", len(dims))
        for d in reversed(dims):
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", gtype, off)
        off += (len(data) + 31) // 32 * 32
    out += b"\0" * ((-len(out)) % 32)
    for _, _, _, data in tensors:
        out += data + b"\0" * ((-len(data)) % 32)
    with open(path, "wb") as f:
        f.write(out)

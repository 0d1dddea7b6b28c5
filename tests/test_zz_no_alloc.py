"""greta_cuda_attn_decode_static: decode attention for callers that cannot allocate device memory
and have no scratch buffer to pass (a host that hands out raw pointers from its own fixed pool, or a
serving loop that must never hit cudaMalloc).  The call keeps the per-split partial results and the
per-head tickets of its split-sequence kernel in an array built into the library, and always takes
the scratch-merge kernel (the cluster kernel, the default of greta_cuda_attn_decode, needs no scratch).

Checked here through the C ABI against the CPU oracle and against greta_cuda_attn_decode forced onto
the same scratch-merge kernel with caller-provided scratch, on calls in a row whose head counts,
head sizes and lengths differ: every call after the first finds the leftovers of a differently shaped
call in the shared array.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import numpy as np
import pytest

from _support import load_package, max_abs_rel
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def g():
    pkg = load_package()
    pkg.build()
    pkg.ffi.require_device()
    return pkg.ffi


# (heads, kv heads, head dim, keys, cache rows); every shape splits the sequence (more than 64 keys).
CALLS = [(32, 32, 128, 2049, 2304), (64, 8, 128, 700, 1024), (8, 2, 64, 97, 128), (32, 32, 128, 2044, 2304), (64, 8, 128, 695, 1024)]


def test_static_scratch_variant_matches_oracle_and_the_scratch_taking_entry_point(g):
    lib = g.cuda()
    rng = np.random.default_rng(60)
    keep = []
    try:
        for H, Hkv, Dh, L, max_seq in CALLS:                   # calls in a row on the one shared array
            scale = float(1.0 / np.sqrt(Dh))
            k = rng.normal(0, 1, (Hkv, max_seq, Dh)).astype(np.float16).view(np.uint16)
            v = rng.normal(0, 1, (Hkv, max_seq, Dh)).astype(np.float16).view(np.uint16)
            q = rng.normal(0, 1, H * Dh).astype(np.float32)
            kc, vc, qd = g.DeviceBuffer.from_numpy(k), g.DeviceBuffer.from_numpy(v), g.DeviceBuffer.from_numpy(q)
            nbytes = lib.greta_cuda_attn_decode_scratch_bytes(H, Dh)
            scratch = g.DeviceBuffer(nbytes, zero=True)
            sib_o, got_o = g.DeviceBuffer(H * Dh * 4), g.DeviceBuffer(H * Dh * 4)
            keep += [kc, vc, qd, scratch, sib_o, got_o]
            got_o.fill(0xFF)                                    # NaN pattern: an unwritten output is caught
            g.check(lib.greta_cuda_attn_decode_static(None, qd.ptr, kc.ptr, vc.ptr, got_o.ptr, None, L, H, Hkv, Dh, max_seq, scale))
            g.check(lib.greta_cuda_set_tuning(b"attn_cluster", 0))   # the sibling entry on the same kernel, its own scratch
            try:
                g.check(lib.greta_cuda_attn_decode(None, qd.ptr, kc.ptr, vc.ptr, sib_o.ptr, None, L, H, Hkv, Dh, max_seq, scale, scratch.ptr, nbytes))
            finally:
                g.check(lib.greta_cuda_set_tuning(b"attn_cluster", 1))
            g.check(lib.greta_cuda_device_synchronize())
            got, sib = got_o.download(np.float32), sib_o.download(np.float32)
            want = O.attention_decode(q, k, v, H, Hkv, Dh, L, max_seq, scale)
            assert np.isfinite(got).all()
            assert max_abs_rel(got, want) < 1e-5                # the tolerance of the attention parity tests
            assert np.array_equal(got, sib)                     # same kernel, same split sizes, fixed merge order: same bits
    finally:
        for b in keep:
            b.free()


def test_static_scratch_variant_rejects_shapes_beyond_its_array(g):
    lib = g.cuda()
    buf = g.DeviceBuffer(1 << 16)
    rc = lib.greta_cuda_attn_decode_static(None, buf.ptr, buf.ptr, buf.ptr, buf.ptr, None, 4, 128, 128, 128, 16, 1.0)
    assert rc == 4
    assert b"at most 64 heads" in lib.greta_cuda_last_error()

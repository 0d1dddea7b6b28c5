"""greta_cuda_attn_decode_static: decode attention for callers that cannot allocate device memory
and have no scratch buffer to pass (a host that hands out raw pointers from its own fixed pool, or a
serving loop that must never hit cudaMalloc).  The call keeps its split-sequence partial results in an
array built into the library.  Checked here through the C ABI against greta_cuda_attn_decode on the
same inputs, twice in a row (the second call finds the first call's leftovers in the shared array).

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import numpy as np
import pytest

from _support import load_package, max_abs_rel

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def g():
    pkg = load_package()
    pkg.build()
    pkg.ffi.require_device()
    return pkg.ffi


@pytest.mark.parametrize("H,Hkv,Dh,L,max_seq", [(32, 32, 128, 2049, 2304), (64, 8, 128, 700, 1024), (8, 2, 64, 97, 128)])
def test_static_scratch_variant_matches_the_scratch_taking_entry_point(g, H, Hkv, Dh, L, max_seq):
    lib = g.cuda()
    rng = np.random.default_rng(60 + L)
    scale = float(1.0 / np.sqrt(Dh))
    kc = g.DeviceBuffer.from_numpy(rng.normal(0, 1, (Hkv, max_seq, Dh)).astype(np.float16).view(np.uint16))
    vc = g.DeviceBuffer.from_numpy(rng.normal(0, 1, (Hkv, max_seq, Dh)).astype(np.float16).view(np.uint16))
    nbytes = lib.greta_cuda_attn_decode_scratch_bytes(H, Dh)
    scratch = g.DeviceBuffer(nbytes, zero=True)
    want_o, got_o = g.DeviceBuffer(H * Dh * 4), g.DeviceBuffer(H * Dh * 4)
    for call in range(2):                                  # two calls in a row, different queries and lengths
        q = g.DeviceBuffer.from_numpy(rng.normal(0, 1, H * Dh).astype(np.float32))
        length = L - call * 5
        got_o.fill(0xFF)
        g.check(lib.greta_cuda_attn_decode(None, q.ptr, kc.ptr, vc.ptr, want_o.ptr, None, length, H, Hkv, Dh, max_seq, scale,
                                           scratch.ptr, nbytes))
        g.check(lib.greta_cuda_attn_decode_static(None, q.ptr, kc.ptr, vc.ptr, got_o.ptr, None, length, H, Hkv, Dh, max_seq, scale))
        g.check(lib.greta_cuda_device_synchronize())
        want, got = want_o.download(np.float32), got_o.download(np.float32)
        assert np.isfinite(got).all()
        assert max_abs_rel(got, want) < 1e-5               # the tolerance of the attention parity tests


def test_static_scratch_variant_rejects_shapes_beyond_its_array(g):
    lib = g.cuda()
    buf = g.DeviceBuffer(1 << 16)
    rc = lib.greta_cuda_attn_decode_static(None, buf.ptr, buf.ptr, buf.ptr, buf.ptr, None, 4, 128, 128, 128, 16, 1.0)
    assert rc == 4
    assert b"at most 64 heads" in lib.greta_cuda_last_error()

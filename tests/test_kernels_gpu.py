"""Parity of the CUDA kernels with the CPU oracle, through the C ABI, on seeded inputs.

Bars: dequantised values bit-exact; matmul and attention within max-abs-rel 2e-3 of the
double-accumulating oracle (fp32 accumulation on the device).  The observed errors are far
smaller; tighter internal bars are asserted where the arithmetic allows it.
"""
import ctypes as C

import numpy as np
import pytest

from _support import load_package, make_blocks, max_abs_rel, q4_0_blocks
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-3          # north-star tolerance (max-abs-rel, fp32 accumulation)
TIGHT = 2e-5        # what fp32 accumulation against a double oracle actually gives

FMTS = {"q4_0": (O.FMT_Q4_0, 8), "q8_0": (O.FMT_Q8_0, 9)}


@pytest.fixture(scope="module")
def g():
    pkg = load_package()
    pkg.build()
    pkg.ffi.require_device()
    return pkg.ffi


_KEEP = []


@pytest.fixture
def tuning(g):
    """Sets a tuning switch of the library for the duration of a test."""
    undo = []

    def set_(name, value, restore):
        g.check(g.cuda().greta_cuda_set_tuning(name.encode(), value), "set_tuning")
        undo.append((name, restore))

    yield set_
    for name, restore in undo:
        g.cuda().greta_cuda_set_tuning(name.encode(), restore)


@pytest.fixture(autouse=True)
def _release_device_buffers():
    yield
    for b in _KEEP:
        b.free()
    _KEEP.clear()


def _dev(g, arr):
    """Uploads arr; the buffer stays alive until the end of the test (a temporary would be freed,
    and its address reused, before the kernel that reads it has run)."""
    b = g.DeviceBuffer.from_numpy(arr)
    _KEEP.append(b)
    return b


def _nan_buffer(g, n_floats):
    b = g.DeviceBuffer(n_floats * 4)
    b.fill(0xFF)            # NaN pattern: unwritten outputs are caught
    return b


# ----------------------------------------------------------------------------- formats
@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
def test_repack_and_dequant_bit_exact(g, name):
    ofmt, gfmt = FMTS[name]
    rng = np.random.default_rng(11)
    N, K = 37, 352
    blk = make_blocks(rng, ofmt, N, K)
    w = g.Weight(blk, gfmt, N, K)
    out = g.DeviceBuffer(N * K * 4)
    g.check(g.cuda().greta_cuda_dequant(None, gfmt, w.qs.ptr, w.d.ptr, out.ptr, N, K))
    got = out.download(np.float32)
    want = O.dequant(blk, ofmt)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # the planes hold exactly GGUF's bytes: scales first two bytes of each block, payload the rest
    bb = g.GGUF_BLOCK_BYTES[gfmt]
    b2 = blk.reshape(-1, bb)
    nb = K // 32
    nbp = (nb + 7) // 8 * 8                      # scale rows are padded to 8 entries (16 bytes), padding is zero
    assert g.cuda().greta_cuda_d_bytes(gfmt, N, K) == N * nbp * 2
    dplane = w.d.download(np.uint16, N * nbp).reshape(N, nbp)
    assert np.array_equal(dplane[:, :nb].reshape(-1), b2[:, :2].copy().view(np.uint16).reshape(-1))
    assert not dplane[:, nb:].any()
    assert np.array_equal(w.qs.download(np.uint8, b2[:, 2:].size), b2[:, 2:].reshape(-1))


def test_dequant_reference_storage_bit_exact(g):
    rng = np.random.default_rng(12)
    n = 64 * 96
    src = rng.normal(0, 0.02, n).astype(np.float32)
    pk, sc = O.quantize_ref_int4(src)
    out = g.DeviceBuffer(n * 4)
    g.check(g.cuda().greta_cuda_dequant(None, g.FMT_REF_INT4, _dev(g, pk).ptr, _dev(g, sc).ptr, out.ptr, 64, 96))
    assert np.array_equal(out.download(np.float32).view(np.uint32), O.dequant_ref_int4(pk, sc).view(np.uint32))
    w8, s8 = O.quantize_ref_int8(src)
    g.check(g.cuda().greta_cuda_dequant(None, g.FMT_REF_INT8, _dev(g, w8).ptr, _dev(g, s8).ptr, out.ptr, 64, 96))
    assert np.array_equal(out.download(np.float32).view(np.uint32), O.dequant_ref_int8(w8, s8).view(np.uint32))


def test_f16_conversions_bit_exact(g):
    rng = np.random.default_rng(13)
    f = np.concatenate([rng.normal(0, 1, 4099), rng.normal(0, 1e-5, 4096), rng.normal(0, 1e-7, 1024),
                        [0.0, -0.0, 65504.0, 65520.0, 1e9, -1e9]]).astype(np.float32)
    src = _dev(g, f)
    dst = g.DeviceBuffer(f.size * 2)
    g.check(g.cuda().greta_cuda_f32_to_f16(None, src.ptr, dst.ptr, f.size))
    bits = dst.download(np.uint16)
    assert np.array_equal(bits, O.f32_to_f16_bits(f))
    back = g.DeviceBuffer(f.size * 4)
    g.check(g.cuda().greta_cuda_f16_to_f32(None, dst.ptr, back.ptr, f.size))
    assert np.array_equal(back.download(np.float32).view(np.uint32), O.f16_bits_to_f32(bits).view(np.uint32))


# ----------------------------------------------------------------------------- GEMV
GEMV_SHAPES = [(1, 1, 32), (1, 3, 64), (1, 17, 96), (2, 5, 1056), (1, 257, 4096), (3, 130, 2048), (1, 64, 11008),
               (1, 4100, 512)]


@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
@pytest.mark.parametrize("M,N,K", GEMV_SHAPES)
def test_gemv_matches_oracle(g, name, M, N, K):
    ofmt, gfmt = FMTS[name]
    rng = np.random.default_rng(100 + N + K)
    blk = make_blocks(rng, ofmt, N, K)
    x = rng.normal(0, 1, (M, K)).astype(np.float32)
    w = g.Weight(blk, gfmt, N, K)
    y = _nan_buffer(g, M * N)
    g.check(g.cuda().greta_cuda_gemv(None, gfmt, _dev(g, x).ptr, 0, w.qs.ptr, w.d.ptr, y.ptr, M, N, K))
    got = y.download(np.float32).reshape(M, N)
    want = O.gemv(x, blk, ofmt, N, K, O.ACC_F64)
    assert np.isfinite(got).all()
    err = max_abs_rel(got, want)
    assert err < TOL and err < TIGHT, err


def test_gemv_fp16_activations(g):
    """The reference instantiates its INT4 GEMV for fp16 activations too (gemm_kernels.hip:921-925)."""
    rng = np.random.default_rng(5)
    N, K = 96, 1024
    blk = q4_0_blocks(rng, N, K)
    xh = rng.normal(0, 1, K).astype(np.float16)
    w = g.Weight(blk, g.FMT_Q4_0, N, K)
    y = _nan_buffer(g, N)
    g.check(g.cuda().greta_cuda_gemv(None, g.FMT_Q4_0, _dev(g, xh.view(np.uint16)).ptr, 1, w.qs.ptr, w.d.ptr, y.ptr, 1, N, K))
    want = O.gemv(xh.view(np.uint16).reshape(1, K), blk, O.FMT_Q4_0, N, K)
    assert max_abs_rel(y.download(np.float32), want[0]) < TIGHT


def test_gemv_reference_int4_int8_storage(g):
    """The reference's own INT4 / INT8 planes (fp32 scales, adjacent-nibble packing) give the same
    products as the oracle's dequantised weights."""
    rng = np.random.default_rng(6)
    N, K = 70, 1312
    src = rng.normal(0, 0.02, N * K).astype(np.float32)
    x = rng.normal(0, 1, K).astype(np.float32)
    for gfmt, (planes, deq) in {g.FMT_REF_INT4: (O.quantize_ref_int4(src), O.dequant_ref_int4),
                                g.FMT_REF_INT8: (O.quantize_ref_int8(src), O.dequant_ref_int8)}.items():
        wq, sc = planes
        W = deq(wq, sc).reshape(N, K).astype(np.float64)
        y = _nan_buffer(g, N)
        g.check(g.cuda().greta_cuda_gemv(None, gfmt, _dev(g, x).ptr, 0, _dev(g, wq).ptr, _dev(g, sc).ptr, y.ptr, 1, N, K))
        assert max_abs_rel(y.download(np.float32), W @ x.astype(np.float64)) < TIGHT


def test_gemv_f16_weights_lm_head_form(g):
    rng = np.random.default_rng(7)
    N, K = 1003, 512
    W = rng.normal(0, 0.02, (N, K)).astype(np.float16)
    x = rng.normal(0, 1, (2, K)).astype(np.float32)
    y = _nan_buffer(g, 2 * N)
    g.check(g.cuda().greta_cuda_gemv(None, g.FMT_F16, _dev(g, x).ptr, 0, _dev(g, W.view(np.uint16)).ptr, None, y.ptr, 2, N, K))
    want = O.gemm_f16w(x, W.view(np.uint16), N, K)
    assert max_abs_rel(y.download(np.float32).reshape(2, N), want) < TIGHT


def test_gemv_linearity_at_full_size(g):
    """Size-independent property at the FFN projection shape of the 7B model (11008 x 4096, Q4_0): W(a x1 + b x2) = a W x1 + b W x2,
    and a sampled row check against the oracle."""
    rng = np.random.default_rng(8)
    N, K = 11008, 4096
    blk = q4_0_blocks(rng, N, K)
    w = g.Weight(blk, g.FMT_Q4_0, N, K)
    x1 = rng.normal(0, 1, K).astype(np.float32)
    x2 = rng.normal(0, 1, K).astype(np.float32)
    xs = np.stack([x1, x2, (0.5 * x1.astype(np.float64) - 2.0 * x2.astype(np.float64)).astype(np.float32)])
    y = _nan_buffer(g, 3 * N)
    g.check(g.cuda().greta_cuda_gemv(None, g.FMT_Q4_0, _dev(g, xs).ptr, 0, w.qs.ptr, w.d.ptr, y.ptr, 3, N, K))
    got = y.download(np.float32).reshape(3, N).astype(np.float64)
    assert np.abs(got[2] - (0.5 * got[0] - 2.0 * got[1])).max() / np.abs(got[2]).max() < 1e-5
    rows = rng.choice(N, 64, replace=False)
    bb = 18 * (K // 32)
    sub = np.concatenate([blk[r * bb:(r + 1) * bb] for r in rows])
    want = O.gemv(x1, sub, O.FMT_Q4_0, 64, K)
    assert max_abs_rel(got[0][rows], want[0]) < TIGHT


@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
def test_gemv_residual(g, name):
    ofmt, gfmt = FMTS[name]
    rng = np.random.default_rng(9)
    N, K = 515, 1408
    blk = make_blocks(rng, ofmt, N, K)
    x = rng.normal(0, 1, K).astype(np.float32)
    r = rng.normal(0, 1, N).astype(np.float32)
    w = g.Weight(blk, gfmt, N, K)
    rb = _dev(g, r)
    g.check(g.cuda().greta_cuda_gemv_residual(None, gfmt, _dev(g, x).ptr, w.qs.ptr, w.d.ptr, rb.ptr, rb.ptr, N, K))  # in place
    want = r.astype(np.float64) + O.gemv(x, blk, ofmt, N, K)[0]
    assert max_abs_rel(rb.download(np.float32), want) < TIGHT


# ----------------------------------------------------------------------------- fused decode operators
@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
@pytest.mark.parametrize("H,Hkv,Dh,D,pos", [(4, 4, 128, 512, 0), (8, 2, 64, 256, 37), (32, 32, 128, 4096, 2047)])
def test_fused_rmsnorm_qkv_rope_kv(g, name, H, Hkv, Dh, D, pos):
    if name == "q8_0" and D == 4096:
        pytest.skip("large case covered by q4_0")
    ofmt, gfmt = FMTS[name]
    rng = np.random.default_rng(20 + H + pos)
    max_seq = pos + 3
    x = rng.normal(0, 1, D).astype(np.float32)
    gamma = rng.normal(1, 0.1, D).astype(np.float32)
    bq, bk, bv = (make_blocks(rng, ofmt, n, D) for n in (H * Dh, Hkv * Dh, Hkv * Dh))
    wq, wk, wv = g.Weight(bq, gfmt, H * Dh, D), g.Weight(bk, gfmt, Hkv * Dh, D), g.Weight(bv, gfmt, Hkv * Dh, D)
    q_out, k_out, v_out = _nan_buffer(g, H * Dh), _nan_buffer(g, Hkv * Dh), _nan_buffer(g, Hkv * Dh)
    kc = g.DeviceBuffer(Hkv * max_seq * Dh * 2, zero=True)
    vc = g.DeviceBuffer(Hkv * max_seq * Dh * 2, zero=True)
    dpos = _dev(g, np.array([pos], np.uint32))
    g.check(g.cuda().greta_cuda_fused_rmsnorm_qkv_rope_kv(
        None, gfmt, _dev(g, x).ptr, _dev(g, gamma).ptr, 1e-5, wq.qs.ptr, wq.d.ptr, wk.qs.ptr, wk.d.ptr, wv.qs.ptr, wv.d.ptr,
        q_out.ptr, k_out.ptr, v_out.ptr, kc.ptr, vc.ptr, dpos.ptr, H, Hkv, Dh, max_seq, 10000.0, D))
    xn = O.rmsnorm(x.reshape(1, D), gamma, 1e-5)
    q = O.rope(O.gemv(xn, bq, ofmt, H * Dh, D), 1, H, Dh, 10000.0, pos).ravel()
    k = O.rope(O.gemv(xn, bk, ofmt, Hkv * Dh, D), 1, Hkv, Dh, 10000.0, pos).ravel()
    v = O.gemv(xn, bv, ofmt, Hkv * Dh, D).ravel()
    # RoPE at large positions amplifies the 1-ulp differences of powf/cosf/sinf between libm and the device
    bar = 5e-4
    assert max_abs_rel(q_out.download(np.float32), q) < bar
    assert max_abs_rel(k_out.download(np.float32), k) < bar
    assert max_abs_rel(v_out.download(np.float32), v) < TIGHT
    kc_h = kc.download(np.uint16).reshape(Hkv, max_seq, Dh)
    vc_h = vc.download(np.uint16).reshape(Hkv, max_seq, Dh)
    # the cache row holds the fp16 rounding of exactly what was returned in fp32
    assert np.array_equal(kc_h[:, pos, :].ravel(), O.f32_to_f16_bits(k_out.download(np.float32)))
    assert np.array_equal(vc_h[:, pos, :].ravel(), O.f32_to_f16_bits(v_out.download(np.float32)))
    other = np.ones(max_seq, bool)
    other[pos] = False
    assert not kc_h[:, other, :].any() and not vc_h[:, other, :].any()      # no other row touched


@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
@pytest.mark.parametrize("D,F", [(256, 34), (512, 1377), (4096, 11008)])
def test_fused_ffn_front(g, name, D, F):
    if name == "q8_0" and D == 4096:
        pytest.skip("large case covered by q4_0")
    ofmt, gfmt = FMTS[name]
    rng = np.random.default_rng(30 + F)
    x = rng.normal(0, 1, D).astype(np.float32)
    gamma = rng.normal(1, 0.1, D).astype(np.float32)
    b1, b3 = make_blocks(rng, ofmt, F, D), make_blocks(rng, ofmt, F, D)
    w1, w3 = g.Weight(b1, gfmt, F, D), g.Weight(b3, gfmt, F, D)
    y = _nan_buffer(g, F)
    g.check(g.cuda().greta_cuda_fused_ffn_front(None, gfmt, _dev(g, x).ptr, _dev(g, gamma).ptr, 1e-5, w1.qs.ptr, w1.d.ptr,
                                                w3.qs.ptr, w3.d.ptr, y.ptr, D, F))
    xn = O.rmsnorm(x.reshape(1, D), gamma, 1e-5)
    want = O.silu_mul(O.gemv(xn, b1, ofmt, F, D), O.gemv(xn, b3, ofmt, F, D)).ravel()
    assert max_abs_rel(y.download(np.float32), want) < TIGHT


# ----------------------------------------------------------------------------- tensor-parallel exchange (one GPU)
def _exchange(g, tp, rank, slot_ptrs):
    from gretacore_v3_b200.model import PeerExchange
    ex = PeerExchange()
    ex.tp, ex.rank = tp, rank
    for j, ptr in enumerate(slot_ptrs):
        ex.slots[j] = ptr
    return ex


@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
@pytest.mark.parametrize("tp", [1, 2, 3, 8])
def test_fused_exchange_operators_on_one_gpu(g, name, tp):
    """The fused tensor-parallel exchange with every 'rank' on this GPU: tp row-parallel projections (columns of W
    split in whole blocks) scatter their tagged partials into tp slot buffers, one after the other; then each
    rank's consumer (fused FFN front, fused QKV) must see x + the sum of the partials, write it to x_out, and
    compute on it what the plain operators compute.  Two exchanges (both halves of the slot buffer) at one position."""
    lib = g.cuda()
    ofmt, gfmt = FMTS[name]
    rng = np.random.default_rng(70 + tp)
    D, Kfull, F, H, Hkv, Dh, pos, max_seq = 512, 96 * tp, 200, 4, 2, 64, 5, 8
    x = rng.normal(0, 1, D).astype(np.float32)
    a = rng.normal(0, 1, Kfull).astype(np.float32)
    gamma = rng.normal(1, 0.1, D).astype(np.float32)
    wo = make_blocks(rng, ofmt, D, Kfull)
    b1, b3 = make_blocks(rng, ofmt, F, D), make_blocks(rng, ofmt, F, D)
    bq, bk, bv = (make_blocks(rng, ofmt, n, D) for n in (H * Dh, Hkv * Dh, Hkv * Dh))
    bb = wo.size // (D * (Kfull // 32))                       # bytes per GGUF block
    shards = [np.ascontiguousarray(wo.reshape(D, Kfull // 32, bb)[:, r * 3:(r + 1) * 3]).reshape(-1) for r in range(tp)]
    slots = [g.DeviceBuffer(lib.greta_cuda_peer_slot_bytes(tp, D), zero=True) for _ in range(tp)]
    _KEEP.extend(slots)
    dpos = _dev(g, np.array([pos], np.uint32))
    xd, gd = _dev(g, x), _dev(g, gamma)
    w1, w3 = g.Weight(b1, gfmt, F, D), g.Weight(b3, gfmt, F, D)
    wq, wk, wv = g.Weight(bq, gfmt, H * Dh, D), g.Weight(bk, gfmt, Hkv * Dh, D), g.Weight(bv, gfmt, Hkv * Dh, D)
    keep = [w1, w3, wq, wk, wv]                               # weights stay alive until the end of the test
    x_sum = x.astype(np.float64) + O.gemv(a, wo, ofmt, D, Kfull)[0]
    for idx in (0, 1):                                        # exchange 0 feeds the FFN front, exchange 1 the QKV operator
        for r in range(tp):                                   # the producers of all ranks, one after the other
            ws = g.Weight(shards[r], gfmt, D, 96)
            keep.append(ws)
            ex = _exchange(g, tp, r, [b.ptr for b in slots])
            g.check(lib.greta_cuda_gemv_peer_scatter(None, gfmt, _dev(g, a[r * 96:(r + 1) * 96]).ptr, ws.qs.ptr, ws.d.ptr, C.byref(ex), idx,
                                                     dpos.ptr, D, 96))
        for r in range(tp):                                   # every rank's consumer reads its own slot buffer
            ex = _exchange(g, tp, r, [b.ptr for b in slots])
            x_out = _nan_buffer(g, D)
            _KEEP.append(x_out)
            if idx == 0:
                y = _nan_buffer(g, F)
                g.check(lib.greta_cuda_fused_ffn_front_peer(None, gfmt, xd.ptr, x_out.ptr, C.byref(ex), idx, dpos.ptr, gd.ptr, 1e-5, w1.qs.ptr,
                                                            w1.d.ptr, w3.qs.ptr, w3.d.ptr, y.ptr, D, F))
                got_x = x_out.download(np.float32)
                xn = O.rmsnorm(got_x.reshape(1, D), gamma, 1e-5)
                want = O.silu_mul(O.gemv(xn, b1, ofmt, F, D), O.gemv(xn, b3, ofmt, F, D)).ravel()
                assert max_abs_rel(y.download(np.float32), want) < TIGHT
            else:
                q_out = _nan_buffer(g, H * Dh)
                kc = g.DeviceBuffer(Hkv * max_seq * Dh * 2, zero=True)
                vc = g.DeviceBuffer(Hkv * max_seq * Dh * 2, zero=True)
                g.check(lib.greta_cuda_fused_rmsnorm_qkv_rope_kv_peer(
                    None, gfmt, xd.ptr, x_out.ptr, C.byref(ex), idx, gd.ptr, 1e-5, wq.qs.ptr, wq.d.ptr, wk.qs.ptr, wk.d.ptr, wv.qs.ptr,
                    wv.d.ptr, q_out.ptr, kc.ptr, vc.ptr, dpos.ptr, H, Hkv, Dh, max_seq, 10000.0, D))
                got_x = x_out.download(np.float32)
                xn = O.rmsnorm(got_x.reshape(1, D), gamma, 1e-5)
                q = O.rope(O.gemv(xn, bq, ofmt, H * Dh, D), 1, H, Dh, 10000.0, pos).ravel()
                assert max_abs_rel(q_out.download(np.float32), q) < 5e-4
                v = O.gemv(xn, bv, ofmt, Hkv * Dh, D).ravel()
                assert max_abs_rel(O.f16_bits_to_f32(vc.download(np.uint16).reshape(Hkv, max_seq, Dh)[:, pos, :].ravel()), v) < 1e-3   # fp16 cache row
            assert max_abs_rel(got_x, x_sum) < TIGHT           # residual stream + sum of the partials
            if r:
                assert np.array_equal(got_x, first_x)          # bit-identical on every rank
            first_x = got_x
    code = C.c_int(-1)
    g.check(lib.greta_cuda_peer_status(C.byref(code)))
    assert code.value == 0


def test_fused_exchange_rejects_bad_descriptors(g):
    lib = g.cuda()
    buf = g.DeviceBuffer(1 << 16, zero=True)
    ok = _exchange(g, 1, 0, [buf.ptr])
    args = (None, g.FMT_Q4_0, buf.ptr, buf.ptr, buf.ptr)
    assert lib.greta_cuda_gemv_peer_scatter(*args, None, 0, buf.ptr, 64, 64) == 4                              # no descriptor
    assert lib.greta_cuda_gemv_peer_scatter(*args, C.byref(ok), 0, None, 64, 64) == 4                          # no position
    assert lib.greta_cuda_gemv_peer_scatter(*args, C.byref(_exchange(g, 9, 0, [buf.ptr])), 0, buf.ptr, 64, 64) == 4   # tp > 8
    assert lib.greta_cuda_gemv_peer_scatter(*args, C.byref(_exchange(g, 2, 0, [buf.ptr])), 0, buf.ptr, 64, 64) == 4   # missing slot buffer
    assert lib.greta_cuda_gemv_peer_scatter(*args, C.byref(ok), 256, buf.ptr, 64, 64) == 4                     # exchange index
    assert lib.greta_cuda_gemv_peer_scatter(None, g.FMT_F16, buf.ptr, buf.ptr, None, C.byref(ok), 0, buf.ptr, 64, 64) == 4   # format
    assert lib.greta_cuda_fused_ffn_front_peer(None, g.FMT_Q4_0, buf.ptr, buf.ptr, C.byref(ok), 0, buf.ptr, buf.ptr, 1e-5, buf.ptr, buf.ptr,
                                               buf.ptr, buf.ptr, buf.ptr, 64, 64) == 4                         # x_out aliases x_in


def test_peer_allreduce_protocol_on_one_gpu(g, tuning):
    """greta_cuda_peer_allreduce_f32 as rank 0 of 2, the other rank played by the host: with nothing from rank 1 the bounded
    waits run out, the status word says so and the call returns; after a reset and with rank 1's tagged words in place
    (its partial of slice 0 in region A, its sums of slice 1 in region B, written by the host with the tag the kernel
    derives from the position) the vector comes back as the sum over both ranks, and rank 0's own words sit where rank 1
    would look for them.  With one rank the call is the identity."""
    import time
    from gretacore_v3_b200.model import PeerExchange
    lib = g.cuda()
    rng = np.random.default_rng(91)
    count, tp, pos, idx = 5 * 512, 2, 7, 3
    slice_ = count // tp
    nbytes = lib.greta_cuda_peer_allreduce_slot_bytes(count)
    assert nbytes == 4 * count * 8
    slots = [g.DeviceBuffer(nbytes, zero=True) for _ in range(tp)]
    _KEEP.extend(slots)
    ex = PeerExchange()
    ex.tp, ex.rank, ex.slot_bytes = tp, 0, nbytes
    for j, b in enumerate(slots):
        ex.slots[j] = b.ptr
    dpos = _dev(g, np.array([pos], np.uint32))
    x0, x1 = rng.normal(0, 1, count).astype(np.float32), rng.normal(0, 1, count).astype(np.float32)
    tag = ((pos + 1) << 8) | idx
    set_off = (idx & 1) * 2 * count

    def run(xbuf):
        g.check(lib.greta_cuda_peer_allreduce_f32(None, xbuf.ptr, count, C.byref(ex), idx, dpos.ptr))
        g.check(lib.greta_cuda_device_synchronize())
        code = C.c_int(-1)
        g.check(lib.greta_cuda_peer_status(C.byref(code)))
        return code.value

    tuning("peer_poll_limit", 2000, restore=1 << 22)
    g.check(lib.greta_cuda_peer_reset(None))
    xd = _dev(g, x0)
    t0 = time.time()
    assert run(xd) != 0 and time.time() - t0 < 5.0              # rank 1 never wrote: the waits gave up by themselves
    # rank 1's part, written by the host into rank 0's buffer
    g.check(lib.greta_cuda_peer_reset(None))
    words = np.zeros((4 * count, 2), np.uint32)
    words[set_off + 1 * slice_: set_off + 2 * slice_, 0] = x1[:slice_].view(np.uint32)             # region A, row 1: rank 1's slice 0
    words[set_off + 1 * slice_: set_off + 2 * slice_, 1] = tag
    total = x0 + x1                                                                                 # rank order: rank 0 first
    words[set_off + count + slice_: set_off + 2 * count, 0] = total[slice_:].view(np.uint32)       # region B, slice 1: summed by rank 1
    words[set_off + count + slice_: set_off + 2 * count, 1] = tag
    slots[0].upload(words.reshape(-1))
    xd = _dev(g, x0)
    assert run(xd) == 0
    assert np.array_equal(xd.download(np.float32), total)
    theirs = slots[1].download(np.uint32).reshape(-1, 2)                                            # what rank 1 would read
    assert np.array_equal(theirs[set_off: set_off + slice_, 0].view(np.float32), x0[slice_:]) and (theirs[set_off: set_off + slice_, 1] == tag).all()
    assert np.array_equal(theirs[set_off + count: set_off + count + slice_, 0].view(np.float32), total[:slice_])
    # one rank: identity, whatever the parity
    ex1 = PeerExchange()
    ex1.tp, ex1.rank, ex1.slot_bytes = 1, 0, nbytes
    ex1.slots[0] = slots[1].ptr
    for i in (0, 1, 2):
        xd = _dev(g, x1)
        g.check(lib.greta_cuda_peer_allreduce_f32(None, xd.ptr, count, C.byref(ex1), i, dpos.ptr))
        g.check(lib.greta_cuda_device_synchronize())
        assert np.array_equal(xd.download(np.float32), x1)
    # refused: slot buffers too small for the count, a count that does not split over the ranks
    ex.slot_bytes = nbytes - 8
    assert lib.greta_cuda_peer_allreduce_f32(None, xd.ptr, count, C.byref(ex), 0, dpos.ptr) != 0
    ex.slot_bytes = nbytes
    assert lib.greta_cuda_peer_allreduce_f32(None, xd.ptr, count - 1, C.byref(ex), 0, dpos.ptr) != 0


def test_fused_exchange_wait_runs_out_and_recovers(g, tuning):
    """A consumer whose producers never ran: with a poll limit of a few thousand the wait gives up by itself, the
    kernel finishes on what it has, greta_cuda_peer_status reports it; after greta_cuda_peer_reset and with the
    partials in place the same call is clean again.  Nothing faults and nothing waits without a bound."""
    import time
    lib = g.cuda()
    ofmt, gfmt = FMTS["q4_0"]
    rng = np.random.default_rng(77)
    tp, D, F, pos = 2, 512, 64, 3
    tuning("peer_poll_limit", 2000, restore=1 << 22)
    g.check(lib.greta_cuda_peer_reset(None))
    slots = [g.DeviceBuffer(lib.greta_cuda_peer_slot_bytes(tp, D), zero=True) for _ in range(tp)]
    _KEEP.extend(slots)
    x, gamma = rng.normal(0, 1, D).astype(np.float32), np.ones(D, np.float32)
    b1, b3 = make_blocks(rng, ofmt, F, D), make_blocks(rng, ofmt, F, D)
    w1, w3 = g.Weight(b1, gfmt, F, D), g.Weight(b3, gfmt, F, D)
    dpos, xd, gd = _dev(g, np.array([pos], np.uint32)), _dev(g, x), _dev(g, gamma)
    x_out, y = _nan_buffer(g, D), _nan_buffer(g, F)
    _KEEP.extend([x_out, y])
    ex = _exchange(g, tp, 0, [b.ptr for b in slots])

    def consume():
        g.check(lib.greta_cuda_fused_ffn_front_peer(None, gfmt, xd.ptr, x_out.ptr, C.byref(ex), 0, dpos.ptr, gd.ptr, 1e-5, w1.qs.ptr, w1.d.ptr,
                                                    w3.qs.ptr, w3.d.ptr, y.ptr, D, F))
        g.check(lib.greta_cuda_device_synchronize())
        code = C.c_int(-1)
        g.check(lib.greta_cuda_peer_status(C.byref(code)))
        return code.value

    t0 = time.time()
    assert consume() != 0                                      # no producer has written: the wait ran out
    assert time.time() - t0 < 5.0                              # and it ran out promptly
    t0 = time.time()
    assert consume() != 0                                      # still flagged: later waits give up at once
    assert time.time() - t0 < 5.0
    # recovery: clear the status, let both producers write, consume again
    g.check(lib.greta_cuda_peer_reset(None))
    a = rng.normal(0, 1, 64 * tp).astype(np.float32)
    wo = make_blocks(rng, ofmt, D, 64 * tp)
    keep = []
    for r in range(tp):
        shard = np.ascontiguousarray(wo.reshape(D, 2 * tp, 18)[:, 2 * r:2 * r + 2]).reshape(-1)
        ws = g.Weight(shard, gfmt, D, 64)
        keep.append(ws)
        exr = _exchange(g, tp, r, [b.ptr for b in slots])
        g.check(lib.greta_cuda_gemv_peer_scatter(None, gfmt, _dev(g, a[r * 64:(r + 1) * 64]).ptr, ws.qs.ptr, ws.d.ptr, C.byref(exr), 0, dpos.ptr,
                                                 D, 64))
    assert consume() == 0
    want_x = x.astype(np.float64) + O.gemv(a, wo, ofmt, D, 64 * tp)[0]
    assert max_abs_rel(x_out.download(np.float32), want_x) < TIGHT


# ----------------------------------------------------------------------------- attention
@pytest.mark.parametrize("H,Hkv,Dh,L,max_seq", [(4, 4, 128, 1, 8), (4, 4, 128, 63, 64), (8, 2, 64, 200, 256),
                                                (32, 32, 128, 2049, 2304), (64, 8, 128, 777, 1024)])
@pytest.mark.parametrize("use_dpos", [False, True])
@pytest.mark.parametrize("cluster", ["1", "0"])
def test_attn_decode_matches_oracle(g, tuning, H, Hkv, Dh, L, max_seq, use_dpos, cluster):
    """Both ways of merging the sequence splits: inside a thread-block cluster through distributed shared memory
    (the default) and through the scratch buffer with tickets (tuning switch attn_cluster = 0)."""
    tuning("attn_cluster", int(cluster), restore=1)
    rng = np.random.default_rng(40 + L)
    q = rng.normal(0, 1, H * Dh).astype(np.float32)
    kc = rng.normal(0, 1, (Hkv, max_seq, Dh)).astype(np.float16)
    vc = rng.normal(0, 1, (Hkv, max_seq, Dh)).astype(np.float16)
    scale = 1.0 / np.sqrt(Dh)
    nbytes = g.cuda().greta_cuda_attn_decode_scratch_bytes(H, Dh)
    scratch = g.DeviceBuffer(nbytes, zero=True)
    o = _nan_buffer(g, H * Dh)
    dpos = _dev(g, np.array([L - 1], np.uint32))
    qd, kd, vd = _dev(g, q), _dev(g, kc.view(np.uint16)), _dev(g, vc.view(np.uint16))
    want = O.attention_decode(q, kc.view(np.uint16), vc.view(np.uint16), H, Hkv, Dh, L, max_seq, scale)
    for _ in range(2):       # twice: the split tickets must be left clean
        o.fill(0xFF)
        g.check(g.cuda().greta_cuda_attn_decode(None, qd.ptr, kd.ptr, vd.ptr, o.ptr, dpos.ptr if use_dpos else None,
                                                0 if use_dpos else L, H, Hkv, Dh, max_seq, scale, scratch.ptr, nbytes))
        got = o.download(np.float32)
        assert np.isfinite(got).all()
        assert max_abs_rel(got, want) < 1e-5
    assert not scratch.download(np.uint32, H).any()


def test_attn_decode_fp32_cache_as_in_the_reference(g):
    rng = np.random.default_rng(41)
    H, Hkv, Dh, L, max_seq = 8, 4, 128, 300, 320
    q = rng.normal(0, 1, H * Dh).astype(np.float32)
    kc = rng.normal(0, 1, (Hkv, max_seq, Dh)).astype(np.float32)
    vc = rng.normal(0, 1, (Hkv, max_seq, Dh)).astype(np.float32)
    nbytes = g.cuda().greta_cuda_attn_decode_scratch_bytes(H, Dh)
    scratch = g.DeviceBuffer(nbytes, zero=True)
    o = _nan_buffer(g, H * Dh)
    g.check(g.cuda().greta_cuda_attn_decode_f32cache(None, _dev(g, q).ptr, _dev(g, kc).ptr, _dev(g, vc).ptr, o.ptr, None, L,
                                                     H, Hkv, Dh, max_seq, 0.0883883, scratch.ptr, nbytes))
    want = O.attention_decode(q, kc, vc, H, Hkv, Dh, L, max_seq, 0.0883883)
    assert max_abs_rel(o.download(np.float32), want) < 1e-5


def test_attn_prefill_causal(g):
    rng = np.random.default_rng(42)
    S, H, Hkv, Dh, max_seq = 70, 8, 4, 64, 96
    q = rng.normal(0, 1, (S, H * Dh)).astype(np.float32)
    k = rng.normal(0, 1, (S, Hkv * Dh)).astype(np.float32)
    v = rng.normal(0, 1, (S, Hkv * Dh)).astype(np.float32)
    kc = g.DeviceBuffer(Hkv * max_seq * Dh * 2, zero=True)
    vc = g.DeviceBuffer(Hkv * max_seq * Dh * 2, zero=True)
    g.check(g.cuda().greta_cuda_kv_update(None, kc.ptr, vc.ptr, _dev(g, k).ptr, _dev(g, v).ptr, S, 0, None, max_seq, Hkv, Dh))
    kc_h = kc.download(np.uint16).reshape(Hkv, max_seq, Dh)
    want_rows = O.f32_to_f16_bits(k).reshape(S, Hkv, Dh).transpose(1, 0, 2)
    assert np.array_equal(kc_h[:, :S, :], want_rows) and not kc_h[:, S:, :].any()
    o = _nan_buffer(g, S * H * Dh)
    scale = 1.0 / np.sqrt(Dh)
    g.check(g.cuda().greta_cuda_attn_prefill(None, _dev(g, q).ptr, kc.ptr, vc.ptr, o.ptr, S, 0, H, Hkv, Dh, max_seq, scale))
    want = O.attention_prefill(q, k, v, S, H, Hkv, Dh, scale, causal=True, kv_round_f16=True)
    assert max_abs_rel(o.download(np.float32).reshape(S, H * Dh), want) < 1e-5


@pytest.mark.parametrize("mma", [1, 0])
@pytest.mark.parametrize("S,pos0,H,Hkv,Dh", [(512, 0, 8, 8, 128), (200, 313, 8, 2, 128), (65, 1, 4, 1, 64), (9, 0, 2, 2, 64)])
def test_attn_prefill_on_tensor_cores_and_on_the_scalar_loop(g, tuning, mma, S, pos0, H, Hkv, Dh):
    """Causal prefill attention of a chunk that starts at pos0 (its queries also see the cache rows of earlier chunks), on
    the tensor-core kernel and on the per-(position, head) loop: every query against the oracle's decode attention over the
    keys 0 .. pos0 + s."""
    tuning("attn_mma", mma, restore=1)
    rng = np.random.default_rng(43 + S)
    max_seq = pos0 + S + 7
    q = rng.normal(0, 1, (S, H * Dh)).astype(np.float32)
    kc = np.zeros((Hkv, max_seq, Dh), np.float16)
    vc = np.zeros((Hkv, max_seq, Dh), np.float16)
    kc[:, :pos0 + S] = rng.normal(0, 1, (Hkv, pos0 + S, Dh)).astype(np.float16)
    vc[:, :pos0 + S] = rng.normal(0, 1, (Hkv, pos0 + S, Dh)).astype(np.float16)
    kc[:, pos0 + S:] = np.float16(100.0)      # rows past the chunk must never be read
    scale = float(1.0 / np.sqrt(Dh))
    o = _nan_buffer(g, S * H * Dh)
    g.check(g.cuda().greta_cuda_attn_prefill(None, _dev(g, q).ptr, _dev(g, kc.view(np.uint16)).ptr, _dev(g, vc.view(np.uint16)).ptr, o.ptr, S, pos0, H,
                                             Hkv, Dh, max_seq, scale))
    got = o.download(np.float32).reshape(S, H * Dh)
    assert np.isfinite(got).all()
    for s_i in sorted({0, 1, 7, 8, 15, 16, 63, 64, S // 2, S - 2, S - 1} & set(range(S))):
        want = O.attention_decode(q[s_i], kc.view(np.uint16), vc.view(np.uint16), H, Hkv, Dh, pos0 + s_i + 1, max_seq, scale)
        assert max_abs_rel(got[s_i], want) < 1e-5, s_i


@pytest.mark.parametrize("use_dpos", [False, True])
def test_rope_matches_oracle(g, use_dpos):
    rng = np.random.default_rng(43)
    S, H, Dh, pos = 5, 6, 128, 1234
    x = rng.normal(0, 1, (S, H * Dh)).astype(np.float32)
    xb = _dev(g, x)
    dpos = _dev(g, np.array([pos], np.uint32))
    g.check(g.cuda().greta_cuda_rope(None, xb.ptr, S, H, Dh, 10000.0, 0 if use_dpos else pos, dpos.ptr if use_dpos else None))
    want = O.rope(x, S, H, Dh, 10000.0, pos)
    assert max_abs_rel(xb.download(np.float32), want.ravel()) < 5e-4


# ----------------------------------------------------------------------------- small operators
def test_rmsnorm_add_silu_mul(g):
    rng = np.random.default_rng(44)
    rows, cols = 3, 4096
    x = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)     # the reference bench's distribution
    gamma = rng.normal(1, 0.1, cols).astype(np.float32)
    y = _nan_buffer(g, rows * cols)
    g.check(g.cuda().greta_cuda_rmsnorm(None, _dev(g, x).ptr, _dev(g, gamma).ptr, y.ptr, rows, cols, 1e-5))
    assert np.allclose(y.download(np.float32).reshape(rows, cols), O.rmsnorm(x, gamma, 1e-5), rtol=1e-5, atol=1e-6)
    a = rng.normal(0, 1, 1000).astype(np.float32)
    b = rng.normal(0, 1, 1000).astype(np.float32)
    c = _nan_buffer(g, 1000)
    g.check(g.cuda().greta_cuda_add(None, _dev(g, a).ptr, _dev(g, b).ptr, c.ptr, 1000))
    assert np.array_equal(c.download(np.float32), a + b)
    g.check(g.cuda().greta_cuda_silu_mul(None, _dev(g, a).ptr, _dev(g, b).ptr, c.ptr, 1000))
    assert np.allclose(c.download(np.float32), O.silu_mul(a, b), rtol=1e-6, atol=1e-7)


def test_embedding_and_argmax(g):
    rng = np.random.default_rng(45)
    vocab, dim = 300, 96
    table = rng.normal(0, 0.02, (vocab, dim)).astype(np.float16)
    toks = np.array([0, 299, 17, -1, 300, 5], np.int32)
    out = _nan_buffer(g, toks.size * dim)
    g.check(g.cuda().greta_cuda_embedding(None, _dev(g, toks).ptr, _dev(g, table.view(np.uint16)).ptr, 1, out.ptr,
                                          toks.size, dim, vocab))
    want = O.embedding(toks, table.view(np.uint16), dim, vocab)
    assert np.array_equal(out.download(np.float32).reshape(toks.size, dim), want)
    assert not want[3].any() and not want[4].any()      # out-of-range ids give zeros
    res = g.DeviceBuffer(4)
    for n in (1, 31, 1024, 32000, 128256):
        logits = rng.normal(0, 1, n).astype(np.float32)
        if n > 100:
            logits[[n // 3, n // 3 + 57 if n // 3 + 57 < n else n - 1]] = 9.5     # an exact tie: first index wins
        g.check(g.cuda().greta_cuda_argmax(None, _dev(g, logits).ptr, n, res.ptr))
        assert int(res.download(np.int32)[0]) == O.argmax(logits)[0] == int(np.argmax(logits))


# ----------------------------------------------------------------------------- prefill GEMM (tcgen05)
def _gemm_status(g):
    code = C.c_int(-1)
    g.check(g.cuda().greta_cuda_gemm_status(C.byref(code)))
    return code.value


@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
@pytest.mark.parametrize("M,N,K,a_f16,c_f16", [(33, 128, 256, True, False), (128, 130, 512, False, False), (130, 200, 256, True, True),
                                               (40, 96, 352, True, False), (200, 4096, 1376, False, False),
                                               (257, 1000, 1024, False, True), (512, 384, 4096, True, True)])
def test_gemm_matches_oracle(g, name, M, N, K, a_f16, c_f16):
    """C = half(A) half(dequant(W))^T: both operands rounded to fp16 as the reference's MFMA route does
    (gemm_kernels.hip:845, 886-887), fp32 accumulation on the tensor cores, against the double-accumulating oracle."""
    ofmt, gfmt = FMTS[name]
    rng = np.random.default_rng(200 + M + N)
    blk = make_blocks(rng, ofmt, N, K)
    a = rng.normal(0, 1, (M, K)).astype(np.float32)
    a_in = a.astype(np.float16).view(np.uint16) if a_f16 else a
    w = g.Weight(blk, gfmt, N, K)
    ws = _KEEP.append(g.DeviceBuffer(g.cuda().greta_cuda_gemm_workspace_bytes(M, K))) or _KEEP[-1]
    c = g.DeviceBuffer(M * N * (2 if c_f16 else 4))
    _KEEP.append(c)
    c.fill(0xFF)
    g.check(g.cuda().greta_cuda_gemm(None, gfmt, _dev(g, a_in).ptr, int(a_f16), w.qs.ptr, w.d.ptr, c.ptr, int(c_f16), M, N, K, ws.ptr))
    g.check(g.cuda().greta_cuda_device_synchronize())
    assert _gemm_status(g) == 0
    if c_f16:
        got = O.f16_bits_to_f32(c.download(np.uint16)).reshape(M, N)
        want = O.f16_bits_to_f32(O.gemm(a_in, blk, ofmt, N, K, out_f16=True))
        bar = 1.5e-3          # one fp16 ulp of the output
    else:
        got = c.download(np.float32).reshape(M, N)
        want = O.gemm(a_in, blk, ofmt, N, K)
        bar = 1e-4            # fp32 accumulation order on the tensor core
    assert np.isfinite(got).all()
    err = max_abs_rel(got, want)
    assert err < TOL and err < bar, err


@pytest.mark.parametrize("tile", ["128x1", "256x1", "512x1", "128x2", "256x2"])
@pytest.mark.parametrize("name,M,N,K", [("q4_0", 600, 300, 1376), ("q8_0", 515, 260, 2048), ("q4_0", 100, 128, 4096)])
def test_gemm_every_tile_shape(g, tuning, name, M, N, K, tile):
    """Every tile shape (tokens x 128-row tiles per CTA, normally chosen from the problem size) gives the same
    product: ragged last token tile, ragged last row tile, odd number of blocks in K, more K stages than any ring is deep."""
    tokens, rows = (int(v) for v in tile.split("x"))
    tuning("gemm_tile", tokens * 10 + rows, restore=0)
    ofmt, gfmt = FMTS[name]
    rng = np.random.default_rng(900 + M + len(tile))
    blk = make_blocks(rng, ofmt, N, K)
    a16 = rng.normal(0, 1, (M, K)).astype(np.float16).view(np.uint16)
    w = g.Weight(blk, gfmt, N, K)
    c = g.DeviceBuffer(M * N * 4)
    _KEEP.append(c)
    c.fill(0xFF)
    g.check(g.cuda().greta_cuda_gemm(None, gfmt, _dev(g, a16).ptr, 1, w.qs.ptr, w.d.ptr, c.ptr, 0, M, N, K, None))
    g.check(g.cuda().greta_cuda_device_synchronize())
    assert _gemm_status(g) == 0
    got = c.download(np.float32).reshape(M, N)
    err = max_abs_rel(got, O.gemm(a16, blk, ofmt, N, K))
    assert np.isfinite(got).all() and err < 1e-4, err


@pytest.mark.parametrize("name,M,N,K,c_f16", [("q4_0", 600, 300, 1376, False), ("q8_0", 515, 260, 2048, False), ("q4_0", 100, 128, 4096, False),
                                              ("q4_0", 257, 1000, 1024, True), ("q8_0", 512, 384, 4096, True), ("q4_0", 1024, 2048, 544, True)])
def test_gemm_cta_pairs(g, tuning, name, M, N, K, c_f16):
    """The two-CTA form (one tcgen05.mma of cta_group::2 per pair, each CTA staging half of the tokens) gives the
    one-CTA product: odd number of row tiles (a CTA with nothing to store), ragged token and row tiles, a second
    token unit that is all padding, odd number of blocks in K, more K stages than the rings are deep, both outputs."""
    tuning("gemm_pair", 2, restore=0)
    ofmt, gfmt = FMTS[name]
    rng = np.random.default_rng(1200 + M + N)
    blk = make_blocks(rng, ofmt, N, K)
    a16 = rng.normal(0, 1, (M, K)).astype(np.float16).view(np.uint16)
    w = g.Weight(blk, gfmt, N, K)
    c = g.DeviceBuffer(M * N * (2 if c_f16 else 4))
    _KEEP.append(c)
    c.fill(0xFF)
    g.check(g.cuda().greta_cuda_gemm(None, gfmt, _dev(g, a16).ptr, 1, w.qs.ptr, w.d.ptr, c.ptr, int(c_f16), M, N, K, None))
    g.check(g.cuda().greta_cuda_device_synchronize())
    assert _gemm_status(g) == 0
    if c_f16:
        got = O.f16_bits_to_f32(c.download(np.uint16)).reshape(M, N)
        want = O.f16_bits_to_f32(O.gemm(a16, blk, ofmt, N, K, out_f16=True))
        bar = 1.5e-3
    else:
        got = c.download(np.float32).reshape(M, N)
        want = O.gemm(a16, blk, ofmt, N, K)
        bar = 1e-4
    assert np.isfinite(got).all()
    err = max_abs_rel(got, want)
    assert err < bar, err
    # and bit for bit what the one-CTA kernel stores (same products, same accumulation order inside the tensor core)
    tuning("gemm_pair", 0, restore=0)
    c1 = g.DeviceBuffer(M * N * (2 if c_f16 else 4))
    _KEEP.append(c1)
    g.check(g.cuda().greta_cuda_gemm(None, gfmt, _dev(g, a16).ptr, 1, w.qs.ptr, w.d.ptr, c1.ptr, int(c_f16), M, N, K, None))
    g.check(g.cuda().greta_cuda_device_synchronize())
    one = c1.download(np.uint16 if c_f16 else np.float32).reshape(M, N)
    two = c.download(np.uint16 if c_f16 else np.float32).reshape(M, N)
    assert max_abs_rel(O.f16_bits_to_f32(two) if c_f16 else two, O.f16_bits_to_f32(one) if c_f16 else one) < 1e-6


@pytest.mark.parametrize("name,M,N,K,a_f16,c_f16", [("q4_0", 512, 1280, 4096, True, True), ("q8_0", 512, 384, 1376, True, False),
                                                    ("q4_0", 1024, 256, 8192, False, False), ("q4_0", 900, 640, 2048, True, True),
                                                    ("q8_0", 512, 1000, 1024, False, True), ("q4_0", 600, 300, 2048, True, False)])
def test_gemm_split_over_k(g, tuning, name, M, N, K, a_f16, c_f16):
    """With fewer 512-token tiles than SMs the K loop of a tile is shared between CTAs: partial sums through the workspace,
    added in ascending K order by the CTA that owns the tile.  Tiles cut into up to eight parts, two token tiles, ragged rows and
    tokens, an odd number of blocks in K, fp32 activations converted into the same workspace, and a shape the plan declines
    (600 tokens: the second token tile would be mostly padding), which must still come out right through the tiled kernel."""
    tuning("gemm_splitk", 2, restore=0)             # 2: wherever the plan is feasible, not only where it is predicted to pay
    ofmt, gfmt = FMTS[name]
    rng = np.random.default_rng(1400 + M + N)
    blk = make_blocks(rng, ofmt, N, K)
    a = rng.normal(0, 1, (M, K)).astype(np.float32)
    a_in = a.astype(np.float16).view(np.uint16) if a_f16 else a
    w = g.Weight(blk, gfmt, N, K)
    ws = g.DeviceBuffer(g.cuda().greta_cuda_gemm_workspace_bytes(M, K))
    _KEEP.append(ws)
    ws.fill(0xEE)                                   # stale bytes in the partial slots and flags must not matter
    c = g.DeviceBuffer(M * N * (2 if c_f16 else 4))
    _KEEP.append(c)
    for rep in range(2):                            # the second launch meets the first launch's flags
        c.fill(0xFF)
        g.check(g.cuda().greta_cuda_gemm(None, gfmt, _dev(g, a_in).ptr, int(a_f16), w.qs.ptr, w.d.ptr, c.ptr, int(c_f16), M, N, K, ws.ptr))
        g.check(g.cuda().greta_cuda_device_synchronize())
        assert _gemm_status(g) == 0
        if c_f16:
            got = O.f16_bits_to_f32(c.download(np.uint16)).reshape(M, N)
            want = O.f16_bits_to_f32(O.gemm(a_in, blk, ofmt, N, K, out_f16=True))
            bar = 1.5e-3
        else:
            got = c.download(np.float32).reshape(M, N)
            want = O.gemm(a_in, blk, ofmt, N, K)
            bar = 1e-4
        assert np.isfinite(got).all()
        err = max_abs_rel(got, want)
        assert err < bar, (rep, err)


def test_gemm_rejects_what_it_cannot_do(g):
    lib = g.cuda()
    buf = g.DeviceBuffer(1 << 16)
    assert lib.greta_cuda_gemm(None, g.FMT_Q4_0, buf.ptr, 1, buf.ptr, buf.ptr, buf.ptr, 0, 64, 64, 48, None) == 4      # K % 32
    assert lib.greta_cuda_gemm(None, g.FMT_F16, buf.ptr, 1, buf.ptr, buf.ptr, buf.ptr, 0, 64, 64, 256, None) == 4     # format
    assert lib.greta_cuda_gemm(None, g.FMT_Q4_0, buf.ptr, 0, buf.ptr, buf.ptr, buf.ptr, 0, 64, 64, 256, None) == 4    # fp32 A without workspace
    assert lib.greta_cuda_gemm(None, g.FMT_Q4_0, None, 1, None, None, None, 0, 0, 64, 256, None) == 0                  # empty

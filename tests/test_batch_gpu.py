"""Batched decode operators (M sequences in step, weights streamed once for all of them) against the CPU oracle
applied row by row, through the C ABI.  The reference has no batch dimension: its arithmetic per sequence is the
single-row path's, which is what the oracle restates.  Bars as for the single-row kernels: matmul max-abs-rel <= 2e-3
(observed ~1e-6: exact integer weight products, activations carried as two fp16 halves), attention < 1e-5."""
import ctypes as C

import numpy as np
import pytest

from _support import load_package, make_blocks, max_abs_rel
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TIGHT = 2e-5
FMTS = {"q4_0": (O.FMT_Q4_0, 8), "q8_0": (O.FMT_Q8_0, 9)}


@pytest.fixture(scope="module")
def g():
    pkg = load_package()
    pkg.build()
    pkg.ffi.require_device()
    return pkg.ffi


_KEEP = []


@pytest.fixture(autouse=True)
def _release():
    yield
    for b in _KEEP:
        b.free()
    _KEEP.clear()


def _dev(g, arr):
    b = g.DeviceBuffer.from_numpy(arr)
    _KEEP.append(b)
    return b


def _ws(g, use, M, K):
    """Workspace for the prepared-activation route, or None for the route that converts inside the matmul kernel."""
    if not use:
        return None
    b = g.DeviceBuffer(g.cuda().greta_cuda_gemv_batch_workspace_bytes(M, K))
    b.fill(0xFF)
    _KEEP.append(b)
    return b.ptr


def _nan(g, n_floats):
    b = g.DeviceBuffer(max(n_floats, 1) * 4)
    b.fill(0xFF)
    _KEEP.append(b)
    return b


@pytest.mark.parametrize("prepared", [True, False])
@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
@pytest.mark.parametrize("M,N,K,slices", [(2, 128, 256, 0), (5, 200, 1376, 1), (16, 384, 2048, 2), (16, 130, 4096, 8), (32, 256, 1024, 4),
                                          (9, 48, 11008, 0), (16, 4096, 4096, 0), (16, 300, 2304, 4), (27, 520, 3584, 2)])
def test_gemv_batch_matches_oracle(g, name, M, N, K, slices, prepared):
    """Plain, with residual, and with the RMSNorm in front; ragged row tiles, K that is not a multiple of the 256-value
    cell, every number of K slices."""
    ofmt, gfmt = FMTS[name]
    lib = g.cuda()
    rng = np.random.default_rng(M * 1000 + N + K)
    blk = make_blocks(rng, ofmt, N, K)
    w = g.Weight(blk, gfmt, N, K)
    x = (rng.normal(0, 1, (M, K)) * rng.uniform(0.01, 30.0, (M, 1))).astype(np.float32)      # rows of very different scale
    x[0, 5:40] = 0.0
    gamma = rng.normal(1, 0.2, K).astype(np.float32)
    resid = rng.normal(0, 1, (M, N)).astype(np.float32)
    xd, gd, rd = _dev(g, x), _dev(g, gamma), _dev(g, resid)
    want = O.gemv(x, blk, ofmt, N, K)
    y = _nan(g, M * N)
    ws = _ws(g, prepared, M, K)
    g.check(lib.greta_cuda_gemv_batch(None, gfmt, xd.ptr, None, 0.0, w.qs.ptr, w.d.ptr, None, y.ptr, M, N, K, slices, ws), "gemv_batch")
    got = y.download(np.float32).reshape(M, N)
    for m in range(M):                                    # per row: a small row must not hide behind a large one
        assert max_abs_rel(got[m], want[m]) < TIGHT, m
    y.fill(0xFF)
    g.check(lib.greta_cuda_gemv_batch(None, gfmt, xd.ptr, None, 0.0, w.qs.ptr, w.d.ptr, rd.ptr, y.ptr, M, N, K, slices, ws), "gemv_batch+resid")
    assert max_abs_rel(y.download(np.float32).reshape(M, N), want.astype(np.float64) + resid) < TIGHT
    y.fill(0xFF)
    g.check(lib.greta_cuda_gemv_batch(None, gfmt, xd.ptr, gd.ptr, 1e-5, w.qs.ptr, w.d.ptr, None, y.ptr, M, N, K, slices, ws), "rmsnorm+gemv_batch")
    wantn = O.gemv(O.rmsnorm(x, gamma, 1e-5), blk, ofmt, N, K)
    got = y.download(np.float32).reshape(M, N)
    for m in range(M):
        assert max_abs_rel(got[m], wantn[m]) < TIGHT, m
    # the general entry point takes the same kernel for 2..32 rows (and loops it above 32)
    y.fill(0xFF)
    g.check(lib.greta_cuda_gemv(None, gfmt, xd.ptr, 0, w.qs.ptr, w.d.ptr, y.ptr, M, N, K), "gemv M>1")
    assert max_abs_rel(y.download(np.float32).reshape(M, N), want) < TIGHT


@pytest.mark.parametrize("prepared", [True, False])
def test_gemv_batch_fp16_weights_lm_head_form(g, prepared):
    lib = g.cuda()
    rng = np.random.default_rng(3)
    M, N, K = 16, 1000, 512
    wbits = rng.normal(0, 0.02, (N, K)).astype(np.float16).view(np.uint16)
    x = rng.normal(0, 1, (M, K)).astype(np.float32)
    gamma = rng.normal(1, 0.1, K).astype(np.float32)
    y = _nan(g, M * N)
    g.check(lib.greta_cuda_gemv_batch(None, g.FMT_F16, _dev(g, x).ptr, _dev(g, gamma).ptr, 1e-5, _dev(g, wbits).ptr, None, None, y.ptr, M, N, K, 0,
                                      _ws(g, prepared, M, K)))
    want = O.gemm_f16w(O.rmsnorm(x, gamma, 1e-5), wbits, N, K)
    assert max_abs_rel(y.download(np.float32).reshape(M, N), want) < TIGHT


def test_gemv_more_than_32_rows_loops_the_batched_kernel(g):
    lib = g.cuda()
    rng = np.random.default_rng(4)
    M, N, K = 45, 96, 512
    blk = make_blocks(rng, O.FMT_Q4_0, N, K)
    w = g.Weight(blk, g.FMT_Q4_0, N, K)
    x = rng.normal(0, 1, (M, K)).astype(np.float32)
    y = _nan(g, M * N)
    g.check(lib.greta_cuda_gemv(None, g.FMT_Q4_0, _dev(g, x).ptr, 0, w.qs.ptr, w.d.ptr, y.ptr, M, N, K))
    assert max_abs_rel(y.download(np.float32).reshape(M, N), O.gemv(x, blk, O.FMT_Q4_0, N, K)) < TIGHT


@pytest.mark.parametrize("prepared", [True, False])
@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
@pytest.mark.parametrize("M,H,Hkv,Dh,D", [(3, 4, 4, 128, 512), (16, 8, 2, 64, 256), (16, 64, 8, 128, 1024)])
def test_fused_qkv_batch(g, name, M, H, Hkv, Dh, D, prepared):
    """Every sequence at its own position: its q is rotated there, its K / V land in that row of its own cache."""
    ofmt, gfmt = FMTS[name]
    lib = g.cuda()
    rng = np.random.default_rng(50 + M + H)
    max_seq = 40
    pos = rng.integers(0, max_seq, M).astype(np.uint32)
    pos[0] = max_seq - 1
    x = rng.normal(0, 1, (M, D)).astype(np.float32)
    gamma = rng.normal(1, 0.1, D).astype(np.float32)
    bq, bk, bv = (make_blocks(rng, ofmt, n, D) for n in (H * Dh, Hkv * Dh, Hkv * Dh))
    wq, wk, wv = g.Weight(bq, gfmt, H * Dh, D), g.Weight(bk, gfmt, Hkv * Dh, D), g.Weight(bv, gfmt, Hkv * Dh, D)
    q_out = _nan(g, M * H * Dh)
    kc = g.DeviceBuffer(M * Hkv * max_seq * Dh * 2, zero=True)
    vc = g.DeviceBuffer(M * Hkv * max_seq * Dh * 2, zero=True)
    _KEEP.extend([kc, vc])
    g.check(lib.greta_cuda_fused_rmsnorm_qkv_rope_kv_batch(None, gfmt, _dev(g, x).ptr, _dev(g, gamma).ptr, 1e-5, wq.qs.ptr, wq.d.ptr, wk.qs.ptr,
                                                           wk.d.ptr, wv.qs.ptr, wv.d.ptr, q_out.ptr, None, None, kc.ptr, vc.ptr, _dev(g, pos).ptr, M,
                                                           H, Hkv, Dh, max_seq, 10000.0, D, _ws(g, prepared, M, D)), "fused_qkv_batch")
    got_q = q_out.download(np.float32).reshape(M, H * Dh)
    got_k = O.f16_bits_to_f32(kc.download(np.uint16)).reshape(M, Hkv, max_seq, Dh)
    got_v = O.f16_bits_to_f32(vc.download(np.uint16)).reshape(M, Hkv, max_seq, Dh)
    for m in range(M):
        xn = O.rmsnorm(x[m:m + 1], gamma, 1e-5)
        q = O.rope(O.gemv(xn, bq, ofmt, H * Dh, D), 1, H, Dh, 10000.0, int(pos[m])).ravel()
        k = O.rope(O.gemv(xn, bk, ofmt, Hkv * Dh, D), 1, Hkv, Dh, 10000.0, int(pos[m])).ravel()
        v = O.gemv(xn, bv, ofmt, Hkv * Dh, D).ravel()
        assert max_abs_rel(got_q[m], q) < 5e-4                                   # RoPE: 1-ulp powf / cosf / sinf differences
        assert max_abs_rel(got_k[m, :, pos[m], :].ravel(), k) < 1e-3             # fp16 cache row
        assert max_abs_rel(got_v[m, :, pos[m], :].ravel(), v) < 1e-3
        other = np.delete(got_k[m], pos[m], axis=1)
        assert not other.any()                                                   # no other row of the cache was touched
    # without positions: no rotation, nothing cached, q / k / v come back
    k_out, v_out = _nan(g, M * Hkv * Dh), _nan(g, M * Hkv * Dh)
    g.check(lib.greta_cuda_fused_rmsnorm_qkv_rope_kv_batch(None, gfmt, _dev(g, x).ptr, None, 0.0, wq.qs.ptr, wq.d.ptr, wk.qs.ptr, wk.d.ptr, wv.qs.ptr,
                                                           wv.d.ptr, q_out.ptr, k_out.ptr, v_out.ptr, None, None, None, M, H, Hkv, Dh, max_seq, 10000.0,
                                                           D, _ws(g, prepared, M, D)), "fused_qkv_batch (plain)")
    assert max_abs_rel(q_out.download(np.float32).reshape(M, -1), O.gemv(x, bq, ofmt, H * Dh, D)) < TIGHT
    assert max_abs_rel(k_out.download(np.float32).reshape(M, -1), O.gemv(x, bk, ofmt, Hkv * Dh, D)) < TIGHT
    assert max_abs_rel(v_out.download(np.float32).reshape(M, -1), O.gemv(x, bv, ofmt, Hkv * Dh, D)) < TIGHT


@pytest.mark.parametrize("prepared", [True, False])
@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
@pytest.mark.parametrize("M,D,F", [(2, 256, 34), (16, 512, 1377), (16, 4096, 11008)])
def test_fused_ffn_front_batch(g, name, M, D, F, prepared):
    ofmt, gfmt = FMTS[name]
    lib = g.cuda()
    rng = np.random.default_rng(60 + M + F)
    x = rng.normal(0, 1, (M, D)).astype(np.float32)
    gamma = rng.normal(1, 0.1, D).astype(np.float32)
    b1, b3 = make_blocks(rng, ofmt, F, D), make_blocks(rng, ofmt, F, D)
    w1, w3 = g.Weight(b1, gfmt, F, D), g.Weight(b3, gfmt, F, D)
    y = _nan(g, M * F)
    g.check(lib.greta_cuda_fused_ffn_front_batch(None, gfmt, _dev(g, x).ptr, _dev(g, gamma).ptr, 1e-5, w1.qs.ptr, w1.d.ptr, w3.qs.ptr, w3.d.ptr, y.ptr,
                                                 M, D, F, _ws(g, prepared, M, D)), "ffn_front_batch")
    xn = O.rmsnorm(x, gamma, 1e-5)
    want = O.silu_mul(O.gemv(xn, b1, ofmt, F, D), O.gemv(xn, b3, ofmt, F, D))
    got = y.download(np.float32).reshape(M, F)
    for m in range(M):
        assert max_abs_rel(got[m], want[m]) < TIGHT, m


@pytest.mark.parametrize("mma", [1, 0])
@pytest.mark.parametrize("M,H,Hkv,Dh,max_seq", [(3, 4, 4, 128, 80), (16, 8, 2, 64, 300), (5, 64, 8, 128, 1100), (16, 8, 1, 128, 700), (4, 32, 2, 128, 200)])
def test_attn_decode_batch(g, M, H, Hkv, Dh, max_seq, mma):
    """Sequences of different lengths (one key up to the whole cache) in one launch; grouped-query shapes take the kernel
    that stages each KV head once for its query heads, the 4/4 shape the per-head kernels."""
    lib = g.cuda()
    g.check(lib.greta_cuda_set_tuning(b"attn_mma", mma))     # grouped-query shapes: tensor-core kernel, or the CUDA-core one
    rng = np.random.default_rng(70 + M + H)
    q = rng.normal(0, 1, (M, H * Dh)).astype(np.float32)
    kc = rng.normal(0, 1, (M, Hkv, max_seq, Dh)).astype(np.float16).view(np.uint16)
    vc = rng.normal(0, 1, (M, Hkv, max_seq, Dh)).astype(np.float16).view(np.uint16)
    pos = rng.integers(0, max_seq, M).astype(np.uint32)
    pos[0], pos[-1] = 0, max_seq - 1
    scale = float(1.0 / np.sqrt(Dh))
    nbytes = lib.greta_cuda_attn_decode_scratch_bytes(M * H, Dh)
    scratch = g.DeviceBuffer(nbytes, zero=True)
    _KEEP.append(scratch)
    o = _nan(g, M * H * Dh)
    qd, kd, vd, pd = _dev(g, q), _dev(g, kc), _dev(g, vc), _dev(g, pos)
    for _ in range(2):
        o.fill(0xFF)
        g.check(lib.greta_cuda_attn_decode_batch(None, qd.ptr, kd.ptr, vd.ptr, o.ptr, pd.ptr, M, H, Hkv, Dh, max_seq, scale, scratch.ptr, nbytes),
                "attn_decode_batch")
        got = o.download(np.float32).reshape(M, H * Dh)
        for m in range(M):
            want = O.attention_decode(q[m], kc[m], vc[m], H, Hkv, Dh, int(pos[m]) + 1, max_seq, scale)
            assert max_abs_rel(got[m], want) < 1e-5, m
    g.check(lib.greta_cuda_set_tuning(b"attn_mma", 1))


def test_argmax_advance_batch(g):
    lib = g.cuda()
    rng = np.random.default_rng(9)
    B, V, cap = 5, 32000, 7
    logits = rng.normal(0, 1, (B, V)).astype(np.float32)
    logits[1, [40, 31999]] = 9.0                                  # a tie: the first maximum wins
    nxt, pos = _dev(g, np.zeros(B, np.int32)), _dev(g, np.arange(10, 10 + B, dtype=np.uint32))
    cnt, outs = _dev(g, np.array([0, 1, 2, 6, 7], np.uint32)), _dev(g, np.full(B * cap, -1, np.int32))
    g.check(lib.greta_cuda_argmax_advance_batch(None, _dev(g, logits).ptr, V, B, nxt.ptr, pos.ptr, outs.ptr, cnt.ptr, cap))
    want = logits.argmax(axis=1)
    assert want[1] == 40
    assert nxt.download(np.int32).tolist() == want.tolist()
    assert pos.download(np.uint32).tolist() == list(range(11, 11 + B))
    assert cnt.download(np.uint32).tolist() == [1, 2, 3, 7, 8]
    got = outs.download(np.int32).reshape(B, cap)
    assert got[0, 0] == want[0] and got[1, 1] == want[1] and got[2, 2] == want[2] and got[3, 6] == want[3]
    assert (got[4] == -1).all()                                   # a full list is left alone


def test_batch_entries_reject_bad_arguments(g):
    lib = g.cuda()
    buf = g.DeviceBuffer(1 << 16)
    _KEEP.append(buf)
    assert lib.greta_cuda_gemv_batch(None, g.FMT_Q4_0, buf.ptr, None, 0.0, buf.ptr, buf.ptr, None, buf.ptr, 33, 64, 64, 0, None) == 4      # M > 32
    assert lib.greta_cuda_gemv_batch(None, g.FMT_Q4_0, buf.ptr, None, 0.0, buf.ptr, buf.ptr, None, buf.ptr, 4, 64, 48, 0, None) == 4       # K % 32
    assert lib.greta_cuda_gemv_batch(None, g.FMT_REF_INT4, buf.ptr, None, 0.0, buf.ptr, buf.ptr, None, buf.ptr, 4, 64, 64, 0, None) == 4   # format
    assert lib.greta_cuda_attn_decode_batch(None, buf.ptr, buf.ptr, buf.ptr, buf.ptr, None, 4, 8, 2, 64, 16, 1.0, None, 0) == 4      # no positions
    assert lib.greta_cuda_fused_rmsnorm_qkv_rope_kv_batch(None, g.FMT_Q4_0, buf.ptr, None, 0.0, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr,
                                                          buf.ptr, None, None, None, None, buf.ptr, 4, 8, 2, 64, 16, 1e4, 64, None) == 4  # positions, no cache

"""CPU-side checks of the boundary: the libraries load and export every symbol the headers
declare, and argument validation answers without touching a GPU."""
import ctypes as C
import os

import pytest

from _support import ROOT, load_package


@pytest.fixture(scope="module")
def pkg():
    p = load_package()
    p.build()
    return p


def test_cuda_library_exports_every_declared_symbol(pkg):
    decls = pkg.ffi.parse_header(os.path.join(ROOT, "include", "greta_cuda.h"))
    names = [d[0] for d in decls]
    assert len(names) >= 45 and len(set(names)) == len(names)
    lib = pkg.ffi.cuda()            # raises AttributeError on a missing export
    for n in names:
        assert hasattr(lib, n)
    for must in ("greta_cuda_gemv", "greta_cuda_gemm", "greta_cuda_fused_rmsnorm_qkv_rope_kv",
                 "greta_cuda_fused_ffn_front", "greta_cuda_attn_decode", "greta_cuda_gemv_residual"):
        assert must in names


def test_size_helpers_need_no_device(pkg):
    lib = pkg.ffi.cuda()
    f = pkg.ffi
    assert lib.greta_cuda_qs_bytes(f.FMT_Q4_0, 4096, 4096) == 4096 * 128 * 16
    assert lib.greta_cuda_d_bytes(f.FMT_Q4_0, 4096, 4096) == 4096 * 128 * 2
    # bytes per weight equal GGUF's: 18/32 and 34/32
    assert lib.greta_cuda_qs_bytes(f.FMT_Q4_0, 11008, 4096) + lib.greta_cuda_d_bytes(f.FMT_Q4_0, 11008, 4096) == 25362432
    assert lib.greta_cuda_qs_bytes(f.FMT_Q8_0, 4096, 4096) + lib.greta_cuda_d_bytes(f.FMT_Q8_0, 4096, 4096) == 17825792
    # scale rows are padded to 16 bytes when K/32 is not a multiple of 8 (tensor-parallel shards of 11008)
    assert lib.greta_cuda_d_bytes(f.FMT_Q4_0, 4096, 1376) == 4096 * 48 * 2
    assert lib.greta_cuda_attn_decode_scratch_bytes(32, 128) > 32 * 4


def test_invalid_arguments_are_rejected_before_any_launch(pkg):
    lib = pkg.ffi.cuda()
    f = pkg.ffi
    buf = (C.c_float * 64)()
    p = C.addressof(buf)
    # K not a multiple of the block size
    assert lib.greta_cuda_gemv(None, f.FMT_Q4_0, p, 0, p, p, p, 1, 4, 48) == 4
    assert b"multiple" in lib.greta_cuda_last_error()
    # unknown format
    assert lib.greta_cuda_gemv(None, 77, p, 0, p, p, p, 1, 4, 64) == 4
    # null pointers
    assert lib.greta_cuda_gemv(None, f.FMT_Q4_0, None, 0, p, p, p, 1, 4, 64) == 4
    assert lib.greta_cuda_gemv_residual(None, f.FMT_Q4_0, p, p, p, None, p, 4, 64) == 4
    # misaligned weight plane
    assert lib.greta_cuda_gemv(None, f.FMT_Q4_0, p, 0, p + 4, p, p, 1, 4, 64) == 4
    # empty problems are silent no-ops like the reference launchers (gemm_kernels.hip:746,915)
    assert lib.greta_cuda_gemv(None, f.FMT_Q4_0, None, 0, None, None, None, 0, 4, 64) == 0
    assert lib.greta_cuda_gemv(None, f.FMT_Q4_0, None, 0, None, None, None, 1, 0, 64) == 0
    # head_dim the attention kernel does not cover
    assert lib.greta_cuda_attn_decode(None, p, p, p, p, None, 1, 4, 4, 96, 16, 1.0, None, 0) in (4, 5)
    assert lib.greta_cuda_attn_decode(None, p, p, p, p, None, 0, 4, 4, 128, 16, 1.0, None, 0) == 4
    assert lib.greta_cuda_fused_rmsnorm_qkv_rope_kv(None, f.FMT_Q4_0, p, p, 1e-5, p, p, p, p, p, p, p, None, None, p, p, p,
                                                    3, 2, 128, 16, 1e4, 64) == 4   # H not a multiple of Hkv


def test_gemm_route_arithmetic():
    """greta_cuda_gemm_route is host arithmetic (no device needed): fixed tiles by default; with the split over K switched on
    and a workspace, shapes with fewer 512-token tiles than SMs share their K loops so that the shares cover every K stage of
    every tile once, a share is never longer than one tile's K loop (a CTA runs at most two segments), and shapes the plan
    declines fall back to tiles."""
    import ctypes as C
    pkg = load_package()
    lib = pkg.ffi.cuda()
    kind, ctas, share, tok = C.c_int(), C.c_uint32(), C.c_uint32(), C.c_uint32()

    def route(M, N, K, ws):
        assert lib.greta_cuda_gemm_route(M, N, K, ws, C.byref(kind), C.byref(ctas), C.byref(share), C.byref(tok)) == 0
        return kind.value, ctas.value, share.value, tok.value

    assert route(512, 11008, 4096, 1) == (0, 86, 64, 512)                 # default: 86 tiles of 512 tokens, 64 K stages each
    assert route(512, 4096, 4096, 0)[0] == 0 and route(512, 4096, 4096, 0)[3] == 128
    assert lib.greta_cuda_set_tuning(b"gemm_splitk", 1) == 0
    try:
        assert route(512, 11008, 4096, 0)[0] == 0                          # no workspace: tiles
        assert route(900, 640, 2048, 1)[0] == 0                            # feasible, but predicted not to pay
        assert lib.greta_cuda_set_tuning(b"gemm_splitk", 2) == 0           # 2: wherever feasible
        assert route(900, 640, 2048, 1)[0] == 2 and route(512, 384, 1376, 1)[0] == 2
        assert route(600, 300, 2048, 1)[0] == 0 and route(4096, 8192, 8192, 1)[0] == 0     # not feasible
        assert lib.greta_cuda_set_tuning(b"gemm_splitk", 1) == 0
        for M, N, K in ((512, 11008, 4096), (512, 4096, 11008), (512, 1024, 8192), (1024, 256, 8192)):
            k, c, s, t = route(M, N, K, 1)
            tiles, kt = ((N + 127) // 128) * ((M + 511) // 512), (K + 63) // 64
            assert k == 2 and t == 512 and s <= kt and c <= 148, (M, N, K, k, c, s)
            assert (c - 1) * s < tiles * kt <= c * s                       # the shares tile the stage units, none is empty
        assert route(600, 300, 2048, 1)[0] == 0                            # second token tile mostly padding: declined
        assert route(4096, 8192, 8192, 1)[0] == 0                          # more tiles than SMs: declined
        assert route(512, 12288, 4096, 1)[0] == 0                          # predicted not to pay: declined
    finally:
        assert lib.greta_cuda_set_tuning(b"gemm_splitk", 0) == 0
    assert lib.greta_cuda_set_tuning(b"gemm_pair", 1) == 0
    try:
        assert route(512, 11008, 4096, 1)[:2] == (1, 86)
        assert route(512, 384, 4096, 1)[0] == 0                            # too few tiles for 512-token tiles: not paired
    finally:
        assert lib.greta_cuda_set_tuning(b"gemm_pair", 0) == 0

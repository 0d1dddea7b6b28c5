"""Pins the CPU oracle against outputs of the reference's own host code.

tests/golden/ref_golden.npz was produced by tests/golden/make_golden.py from the
reference's GGUF loader (weight_loader.cpp), its Buffer class and its header-only
CPU reference (cpu_reference.hpp), compiled from the reference sources.  Where the
compiled reference library is present (oracle/_ref) a few cases also call it live.
"""
import hashlib

import numpy as np
import pytest

from oracle import oracle as O


def test_fp16_decode_matches_reference_for_every_half(golden):
    allh = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    tab = O.f16_bits_to_f32(allh)
    assert np.array_equal(allh[np.isnan(tab)], golden["h2f_nan_bits"])
    tab = np.where(np.isnan(tab), np.float32(0), tab)
    digest = hashlib.sha256(tab.view(np.uint32).tobytes()).digest()
    assert digest == golden["h2f_table_sha256"].tobytes()
    got = O.f16_bits_to_f32(golden["h2f_sample_bits"])
    ok = ~np.isnan(got)
    assert np.array_equal(got.view(np.uint32)[ok], golden["h2f_sample_f32"].view(np.uint32)[ok])
    # numpy's own half decoding agrees too (finite values)
    npy = allh.view(np.float16).astype(np.float32)
    fin = np.isfinite(npy)
    assert np.array_equal(tab[fin], npy[fin])


def test_fp16_encode_matches_reference_on_normal_range(golden):
    f, bits = golden["f2h_in"], golden["f2h_bits"]
    got = O.f32_to_f16_bits(f)
    # The reference's CPU converter truncates subnormal results; the device intrinsic the
    # kernels use rounds them.  The oracle follows the kernels, so compare where the result
    # is normal, zero or infinite.
    normal = (np.abs(f) >= 2.0 ** -14) | (f == 0)
    assert normal.sum() > 3500
    assert np.array_equal(got[normal], bits[normal])
    # and everywhere against IEEE round-to-nearest-even as numpy implements it
    assert np.array_equal(got, f.astype(np.float16).view(np.uint16))


def test_fp16_encode_is_ieee_rne_including_subnormals():
    rng = np.random.default_rng(7)
    f = np.concatenate([rng.normal(0, 1e-5, 20000), rng.normal(0, 1e-7, 20000), rng.normal(0, 1, 20000),
                        rng.normal(0, 4e4, 5000)]).astype(np.float32)
    assert np.array_equal(O.f32_to_f16_bits(f), f.astype(np.float16).view(np.uint16))


def test_int8_quantiser_and_storage_match_reference_loader(golden):
    src = golden["int4_down_src"].ravel()
    w, s = O.quantize_ref_int8(src)
    assert np.array_equal(w, golden["int8_down_w"])
    assert np.array_equal(s.view(np.uint32), golden["int8_down_scales"].view(np.uint32))
    deq = O.dequant_ref_int8(w, s)
    assert np.array_equal(deq, w.astype(np.float32) * np.repeat(s, 32))


def test_q8_0_split_and_dequant_known_answers():
    """Q8_0 {fp16 d; int8 q[32]} -> int8 plane + fp32 scale (weight_loader.cpp:703-712, a branch the
    reference cannot reach at run time, so this is pinned by hand-built blocks)."""
    rng = np.random.default_rng(3)
    nb = 40
    q = rng.integers(-127, 128, (nb, 32), dtype=np.int8)
    d = (np.abs(rng.normal(0, 0.02, nb)) / 127).astype(np.float16)
    d[0], d[1], d[2] = np.float16(6e-8), np.float16(0.0), np.float16(1.5)      # subnormal, zero, normal
    blk = np.empty((nb, 34), np.uint8)
    blk[:, :2] = d.view(np.uint8).reshape(nb, 2)
    blk[:, 2:] = q.view(np.uint8)
    w, s = O.q8_0_split(blk)
    assert np.array_equal(w.reshape(nb, 32), q)
    assert np.array_equal(s, d.astype(np.float32))
    assert (s[3:] < 2.0 ** -14).any()          # the config's scales are largely fp16 subnormals
    expect = q.astype(np.float32) * d.astype(np.float32)[:, None]
    assert np.array_equal(O.dequant(blk, O.FMT_Q8_0).view(np.uint32), expect.ravel().view(np.uint32))
    assert np.array_equal(O.dequant_ref_int8(w, s).view(np.uint32), expect.ravel().view(np.uint32))


@pytest.mark.parametrize("tag", ["attnq", "down"])
def test_int4_quantiser_and_packing_match_reference_loader(golden, tag):
    src = golden[f"int4_{tag}_src"]
    packed, scales = O.quantize_ref_int4(src.ravel())
    assert np.array_equal(packed, golden[f"int4_{tag}_packed"])
    assert np.array_equal(scales.view(np.uint32), golden[f"int4_{tag}_scales"].view(np.uint32))
    # nibble order and sign extension: element 2j low nibble, 2j+1 high nibble, two's complement
    deq = O.dequant_ref_int4(packed, scales)
    lo = (packed & 0xF).astype(np.int8)
    hi = (packed >> 4).astype(np.int8)
    lo[lo > 7] -= 16
    hi[hi > 7] -= 16
    v = np.stack([lo, hi], 1).ravel().astype(np.float32)
    assert np.array_equal(deq, v * np.repeat(scales, 32))
    # quantisation error is bounded by half a step where the scale is non-zero
    step = np.repeat(scales, 32)
    assert np.all(np.abs(deq - src.ravel()) <= 0.5 * step * (1 + 1e-5) + 1e-12)


def test_reference_per_head_scales_are_max_abs(golden):
    src = golden["int4_attnq_src"]
    hs = golden["int4_attnq_head_scales"]
    assert hs.size == 2 and golden["int4_down_head_scales"].size == 0
    assert np.allclose(hs, np.abs(src.reshape(2, -1)).max(1))


def test_q4_0_equals_reference_int4_storage():
    """The GGUF Q4_0 value (q-8)*d maps losslessly onto the reference's INT4 (v=q-8, s=fp32(d))."""
    rng = np.random.default_rng(1)
    nb = 64
    blk = np.empty((nb, 18), np.uint8)
    blk[:, :2] = (np.abs(rng.normal(0, 0.02, nb)) / 8).astype(np.float16).view(np.uint8).reshape(nb, 2)
    blk[:, 2:] = rng.integers(0, 256, (nb, 16), dtype=np.uint8)
    deq = O.dequant(blk, O.FMT_Q4_0)
    packed, scales = O.q4_0_to_ref_int4(blk)
    assert np.array_equal(deq.view(np.uint32), O.dequant_ref_int4(packed, scales).view(np.uint32))
    # hand-built known answer: d = 0.5, qs[j] = j | ((15-j) << 4)
    one = np.zeros(18, np.uint8)
    one[:2] = np.array([0.5], np.float16).view(np.uint8)
    one[2:] = [j | ((15 - j) << 4) for j in range(16)]
    want = np.array([(j - 8) * 0.5 for j in range(16)] + [((15 - j) - 8) * 0.5 for j in range(16)], np.float32)
    assert np.array_equal(O.dequant(one, O.FMT_Q4_0), want)


def test_dense_gemm_matches_cpu_reference(golden):
    A, B, Cm = golden["gemm_A"], golden["gemm_B"], golden["gemm_C"]
    # oracle form: W [N x K] fp16 bits, y = x W^T, double accumulation
    Wbits = np.ascontiguousarray(B.T).astype(np.float16).view(np.uint16)
    got = O.gemm_f16w(A, Wbits, B.shape[1], B.shape[0])
    assert np.array_equal(got.view(np.uint32), Cm.view(np.uint32))
    assert np.array_equal(golden["ka_gemm_C"], np.array([19, 22, 43, 50], np.float32))


def test_rmsnorm_matches_cpu_reference(golden):
    y0 = O.rmsnorm(golden["rms_x"], golden["rms_gamma"], 1e-5, mode=0)
    y1 = O.rmsnorm(golden["rms_x"], golden["rms_gamma"], 1e-5, mode=1)
    assert np.allclose(y0, golden["rms_y"], rtol=3e-7, atol=1e-8)
    assert np.allclose(y1, golden["rms_y"], rtol=2e-6, atol=1e-7)     # the kernel's fp32 order
    ka = O.rmsnorm(np.array([[1, 2, 3, 4]], np.float32), np.ones(4, np.float32), 1e-5)
    assert np.allclose(ka, golden["ka_rms_y"], rtol=3e-7)
    assert np.allclose(ka[0], np.array([1, 2, 3, 4]) / np.sqrt(7.5), atol=1e-5)  # cpu_ref_test.cpp:36-41


@pytest.mark.parametrize("mode,tag", [(0, "fp64"), (1, "fp32")])
def test_attention_matches_the_reference_cpu_attention(golden, mode, tag):
    """oracle_attention_decode against compute_attention_ref_fp64 / _fp32, the CPU references inside the reference's
    block scheduler (src/inference/src/block_scheduler.cpp:721-864): same arithmetic, same order."""
    H, Hkv, Dh, L, S = (int(v) for v in golden["attn_shape"])
    q, k, v, want = golden["attn_q"], golden["attn_k"], golden["attn_v"], golden["attn_out_" + tag]
    got32 = O.attention_decode(q, k, v, H, Hkv, Dh, L, S, 0.125, mode=mode)                     # the reference's fp32 cache
    got16 = O.attention_decode(q, k.astype(np.float16).view(np.uint16), v.astype(np.float16).view(np.uint16), H, Hkv, Dh, L, S, 0.125,
                               mode=mode)                                                        # the same values as an fp16 cache
    assert np.array_equal(got32.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(got16.view(np.uint32), want.view(np.uint32))
    # rows past seq_len are not read: 70 of 80 rows were attended
    k2 = k.copy()
    k2[:, L:] = 1e9
    assert np.array_equal(O.attention_decode(q, k2, v, H, Hkv, Dh, L, S, 0.125, mode=mode), got32)


def test_host_dequantiser_matches_the_reference_read_weight_value(golden):
    """oracle_dequant_ref_int4 / _int8 and the fp16 decoder against read_weight_value
    (src/inference/src/block_scheduler.cpp:639-671) on the planes the reference's own loader produced."""
    got4 = O.dequant_ref_int4(golden["int4_down_packed"], golden["int4_down_scales"])
    assert np.array_equal(got4.view(np.uint32), golden["rwv_int4_down"].view(np.uint32))
    got8 = O.dequant_ref_int8(golden["int8_down_w"], golden["int8_down_scales"])
    assert np.array_equal(got8.view(np.uint32), golden["rwv_int8_down"].view(np.uint32))
    bits = golden["rwv_f16_bits"]
    gotf, want = O.f16_bits_to_f32(bits), golden["rwv_f16"]
    nan_in = ((bits & 0x7C00) == 0x7C00) & ((bits & 0x03FF) != 0)     # that decoder turns fp16 NaNs into infinities; the
    assert np.isinf(want[nan_in]).all() and np.isnan(gotf[nan_in]).all()   # oracle (and the device intrinsic) keep them NaN
    assert np.array_equal(gotf[~nan_in].view(np.uint32), want[~nan_in].view(np.uint32))


def test_live_reference_library_when_present(golden):
    ref = O.ref()
    if ref is None:
        pytest.skip("oracle/_ref not built on this machine (needs the reference checkout)")
    for h in (0x0001, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0x8001, 0xFBFF):
        assert O.lib().oracle_fp16_to_fp32(h) == ref.ref_half_to_float(h)


def test_gemv_accumulation_orders_agree():
    """The kernel's fp32 summation order stays within 1e-5 of the double-accumulating oracle."""
    rng = np.random.default_rng(0)
    N, K = 64, 4096
    x = rng.normal(0, 1, K).astype(np.float32)
    for fmt in (O.FMT_Q4_0, O.FMT_Q8_0):
        bb = O.BLOCK_BYTES[fmt]
        blk = rng.integers(0, 256, (N * K // 32, bb), dtype=np.uint8)
        div = 8 if fmt == O.FMT_Q4_0 else 127
        blk[:, :2] = (np.abs(rng.normal(0, 0.02, len(blk))) / div).astype(np.float16).view(np.uint8).reshape(-1, 2)
        if fmt == O.FMT_Q8_0:
            blk[:, 2:][blk[:, 2:] == 0x80] = 0x81   # q in [-127, 127]
        y64 = O.gemv(x, blk, fmt, N, K, O.ACC_F64)
        yref = O.gemv(x, blk, fmt, N, K, O.ACC_REF_F32)
        yfast = O.gemv(x, blk, fmt, N, K, O.ACC_FAST_F32)
        W = O.dequant(blk, fmt).reshape(N, K).astype(np.float64)
        assert np.allclose(y64[0], W @ x.astype(np.float64), rtol=1e-6, atol=1e-7)
        scale = np.abs(y64).max()
        assert np.abs(yref - y64).max() / scale < 1e-5
        assert np.abs(yfast - y64).max() / scale < 1e-5


@pytest.mark.parametrize("tag", ["q4k", "q6k"])
def test_kquant_decoders_match_the_reference_loader(golden, tag):
    """Q4_K / Q6_K super-blocks decode to the fp32 values GGUFLoader::load_tensor produces, bit for bit
    (weight_loader.cpp:125-177, 520-570), and the decode -> INT4 re-quantisation chain of load_tensor_int4
    (:825-957) gives the reference's packed nibbles and group scales."""
    dec = O.dequant_q4_k if tag == "q4k" else O.dequant_q6_k
    got = dec(golden[tag + "_blocks"])
    assert np.array_equal(got.view(np.uint32), golden[tag + "_f32"].view(np.uint32))
    packed, scales = O.quantize_ref_int4(got)
    assert np.array_equal(packed, golden[tag + "_int4_packed"])
    assert np.array_equal(scales.view(np.uint32), golden[tag + "_int4_scales"].view(np.uint32))


def test_q8_0_quantiser_round_trip():
    """The Q8_0 quantiser K-quant tensors are re-stored with: d = amax / 127 in fp16, |q| <= 127, the largest magnitude
    of a block maps to +-127, and decoding stays within half a step of the input (plus the fp16 rounding of d)."""
    rng = np.random.default_rng(5)
    x = rng.normal(0, 0.03, 64 * 32).astype(np.float32)
    x[32:64] = 0.0                                       # an all-zero block
    blk = O.quantize_q8_0(x).reshape(-1, 34)
    q = blk[:, 2:].view(np.int8).astype(np.int32)
    d = O.f16_bits_to_f32(blk[:, :2].copy().view(np.uint16).reshape(-1))
    xb = x.reshape(-1, 32)
    amax = np.abs(xb).max(axis=1)
    assert np.abs(q).max() <= 127 and (q[1] == 0).all() and d[1] == 0
    assert (np.abs(q).max(axis=1)[amax > 0] == 127).all()
    assert np.array_equal(O.f32_to_f16_bits(amax / np.float32(127.0)), blk[:, :2].copy().view(np.uint16).reshape(-1))
    back = O.dequant(blk, O.FMT_Q8_0).reshape(-1, 32)
    assert (np.abs(back - xb) <= (0.5 + 127 * 2.0 ** -11) * d[:, None] + 1e-12).all()

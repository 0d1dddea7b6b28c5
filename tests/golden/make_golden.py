"""Generates tests/golden/ref_golden.npz by running the reference's OWN host code
(oracle/_ref/libgreta_ref.so, compiled from the reference sources by
`make -C oracle ref`) on small seeded inputs.  Needs the reference checkout, so it
runs only where that exists; the .npz it writes is committed and is what the
CPU tests check the oracle against everywhere else.

    python tests/golden/make_golden.py
"""
import ctypes as C
import hashlib
import os
import struct
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from oracle import oracle  # noqa: E402
from _support import write_gguf  # noqa: E402

GGML_F32, GGML_Q8_0 = 0, 8


def q8_0_blocks(rng, n_blocks, sigma=0.02):
    """GGUF Q8_0 blocks: int8 q uniform in [-127,127], d = |N(0,sigma)|/127 as fp16 (many are subnormal)."""
    q = rng.integers(-127, 128, size=(n_blocks, 32), dtype=np.int8)
    d = (np.abs(rng.normal(0, sigma, n_blocks)) / 127).astype(np.float16)
    blk = np.empty((n_blocks, 34), np.uint8)
    blk[:, :2] = d.view(np.uint8).reshape(n_blocks, 2)
    blk[:, 2:] = q.view(np.uint8)
    return blk


def kquant_blocks(rng, ggml_type, n):
    """Random K-quant super-blocks: every payload, scale and min bit pattern, fp16 super-scales of model-like size
    (one of them subnormal, one zero)."""
    if ggml_type == 12:   # Q4_K: d, dmin, scales[12], qs[128]
        blk = rng.integers(0, 256, (n, 144), dtype=np.uint8)
        d = (np.abs(rng.normal(0, 0.01, (n, 2))) / 16).astype(np.float16)
        d[1, 0] = np.float16(3e-7)
        d[2, 1] = np.float16(0)
        blk[:, :4] = d.view(np.uint8).reshape(n, 4)
    else:                 # Q6_K: ql[128], qh[64], scales[16], d
        blk = rng.integers(0, 256, (n, 210), dtype=np.uint8)
        d = (np.abs(rng.normal(0, 0.01, n)) / 1024).astype(np.float16)
        d[1] = np.float16(2e-7)
        blk[:, 208:] = d.view(np.uint8).reshape(n, 2)
    return blk


def main():
    ref = oracle.ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libgreta_ref.so missing: run `make -C oracle ref` where the reference exists")
    rng = np.random.default_rng(20261125)
    g = {}

    # 1. fp16 -> fp32 over all 65536 bit patterns (CpuReference::half_to_float).
    allh = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    tab = np.array([ref.ref_half_to_float(int(h)) for h in allh], np.float32)
    # NaN payloads do not survive the float -> Python -> float round trip: hash with NaNs zeroed,
    # and keep the NaN positions separately.
    g["h2f_nan_bits"] = allh[np.isnan(tab)].copy()
    tab = np.where(np.isnan(tab), np.float32(0), tab)
    g["h2f_table_sha256"] = np.frombuffer(hashlib.sha256(tab.view(np.uint32).tobytes()).digest(), np.uint8)
    g["h2f_sample_bits"] = allh[::257].copy()
    g["h2f_sample_f32"] = tab[::257].copy()

    # 2. fp32 -> fp16 (CpuReference::float_to_half) on normal-range values and some specials.
    f = np.concatenate([rng.normal(0, 1, 2048), rng.normal(0, 300, 1024), rng.uniform(-7e-5, 7e-5, 1024) + 1e-4,
                        [0.0, -0.0, 1.0, -1.0, 65504.0, 65519.9, 65520.0, 1e6, -1e6, 6.1035156e-05, 0.333251953125,
                         1.00048828125, 1.000732421875, 2049.0, 2051.0]]).astype(np.float32)
    g["f2h_in"] = f
    g["f2h_bits"] = np.array([ref.ref_float_to_half(float(v)) for v in f], np.uint16)

    # 3/4. GGUF file with a Q8_0 tensor and F32 tensors, read back through GGUFLoader.
    dim, heads = 64, 2
    q8 = q8_0_blocks(rng, 8 * dim // 32)                       # tensor [8 x 64]
    wq = rng.normal(0, 0.02, (dim, dim)).astype(np.float32)    # attention tensor -> per-head scales
    wd = rng.normal(0, 0.05, (16, dim)).astype(np.float32)     # plain tensor
    wd[3, :32] = 0.0                                           # an all-zero group (scale 0 path)
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "tiny.gguf")
        write_gguf(path,
                   [("llama.embedding_length", dim), ("llama.attention.head_count", heads),
                    ("llama.attention.head_count_kv", heads), ("llama.block_count", 1),
                    ("llama.feed_forward_length", 128), ("llama.context_length", 256)],
                   [("llama.rope.freq_base", 10000.0), ("llama.norm_eps", 1e-5)],
                   [("blk.0.ffn_gate.weight", [8, dim], GGML_Q8_0, q8.tobytes()),
                    ("blk.0.attn_q.weight", [dim, dim], GGML_F32, wq.tobytes()),
                    ("blk.0.ffn_down.weight", [16, dim], GGML_F32, wd.tobytes())])
        cfg = np.zeros(10, np.uint32)
        assert ref.ref_gguf_config(path.encode(), cfg.ctypes.data_as(C.c_void_p)) == 0
        g["gguf_config"] = cfg
        # GGUFLoader::load_tensor_int8 on an F32 tensor: the reference's INT8 quantiser and storage.
        # (Its Q8_0 branch is unreachable: the loader's type naming has no Q8_0 case, so the Q8_0
        # tensor above is only used to check that the file parses; it is not read back.)
        w8 = np.empty(wd.size, np.int8)
        s8 = np.empty(wd.size // 32, np.float32)
        rc = ref.ref_gguf_load_int8(path.encode(), b"blk.0.ffn_down.weight", w8.ctypes.data_as(C.c_void_p),
                                    C.c_size_t(w8.size), s8.ctypes.data_as(C.c_void_p), C.c_size_t(s8.size))
        assert rc == 0, rc
        g["int8_down_w"], g["int8_down_scales"] = w8, s8
        for tag, name, src in (("attnq", b"blk.0.attn_q.weight", wq), ("down", b"blk.0.ffn_down.weight", wd)):
            pk = np.empty(src.size // 2, np.uint8)
            sc = np.empty(src.size // 32, np.float32)
            hs = np.zeros(heads, np.float32)
            nh = C.c_uint32(0)
            rc = ref.ref_gguf_load_int4(path.encode(), name, pk.ctypes.data_as(C.c_void_p), C.c_size_t(pk.size),
                                        sc.ctypes.data_as(C.c_void_p), C.c_size_t(sc.size),
                                        hs.ctypes.data_as(C.c_void_p), C.c_size_t(hs.size), C.byref(nh))
            assert rc == 0, rc
            g[f"int4_{tag}_src"], g[f"int4_{tag}_packed"], g[f"int4_{tag}_scales"] = src, pk, sc
            g[f"int4_{tag}_head_scales"] = hs[: nh.value].copy()

    # 5. CpuReference dense GEMM (C = A[MxK] * B[KxN], double accumulation) and RMSNorm.
    M, N, K = 5, 7, 96
    A = rng.normal(0, 1, (M, K)).astype(np.float32)
    B = rng.normal(0, 0.05, (K, N)).astype(np.float16).astype(np.float32)  # exactly representable in fp16
    Cm = np.empty((M, N), np.float32)
    ref.ref_cpu_gemm(A.ctypes.data_as(C.c_void_p), B.ctypes.data_as(C.c_void_p), Cm.ctypes.data_as(C.c_void_p), M, N, K)
    g["gemm_A"], g["gemm_B"], g["gemm_C"] = A, B, Cm
    x = rng.uniform(-1, 1, (3, 320)).astype(np.float32)
    gam = rng.normal(1, 0.1, 320).astype(np.float32)
    y = np.empty_like(x)
    ref.ref_cpu_rmsnorm(x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), gam.ctypes.data_as(C.c_void_p),
                        3, 320, C.c_float(1e-5))
    g["rms_x"], g["rms_gamma"], g["rms_y"] = x, gam, y
    # the reference's own known-answer test (tools/bench/runtime/src/cpu_ref_test.cpp:8-42)
    ka = np.array([1, 2, 3, 4], np.float32)
    kb = np.array([5, 6, 7, 8], np.float32)
    kc = np.empty(4, np.float32)
    ref.ref_cpu_gemm(ka.ctypes.data_as(C.c_void_p), kb.ctypes.data_as(C.c_void_p), kc.ctypes.data_as(C.c_void_p), 2, 2, 2)
    g["ka_gemm_C"] = kc
    ky = np.empty(4, np.float32)
    ref.ref_cpu_rmsnorm(ka.ctypes.data_as(C.c_void_p), ky.ctypes.data_as(C.c_void_p),
                        np.ones(4, np.float32).ctypes.data_as(C.c_void_p), 1, 4, C.c_float(1e-5))
    g["ka_rms_y"] = ky

    # 6. The CPU attention references the reference keeps inside its block scheduler
    # (compute_attention_ref_fp64 / _fp32, src/inference/src/block_scheduler.cpp:721-864), GQA 8 / 2 heads of 64,
    # 70 of 80 cache rows.  Cache values are exactly representable in fp16, so the same numbers can be fed to the
    # oracle both as the reference's fp32 cache and as the fp16 cache of the B200 build.
    H, Hkv, Dh, L, S = 8, 2, 64, 70, 80
    aq = rng.normal(0, 1, H * Dh).astype(np.float32)
    ak = rng.normal(0, 1, (Hkv, S, Dh)).astype(np.float16).astype(np.float32)
    av = rng.normal(0, 1, (Hkv, S, Dh)).astype(np.float16).astype(np.float32)
    g["attn_q"], g["attn_k"], g["attn_v"] = aq, ak, av
    g["attn_shape"] = np.array([H, Hkv, Dh, L, S], np.int32)
    for mode, tag in ((0, "fp64"), (1, "fp32")):
        ao = np.empty(H * Dh, np.float32)
        ref.ref_sched_attention(aq.ctypes.data_as(C.c_void_p), ak.ctypes.data_as(C.c_void_p), av.ctypes.data_as(C.c_void_p), H, Hkv, Dh, L, S,
                                C.c_float(0.125), mode, ao.ctypes.data_as(C.c_void_p))
        g["attn_out_" + tag] = ao

    # 7. The reference's host dequantiser read_weight_value (block_scheduler.cpp:639-671) on the INT4 / INT8 planes its
    # own loader produced above, and on fp16 bits.
    def read_weights(dtype, raw, scales, elems):
        raw = np.ascontiguousarray(raw).view(np.uint8)
        o = np.empty(elems, np.float32)
        ref.ref_sched_read_weights(dtype, raw.ctypes.data_as(C.c_void_p), C.c_size_t(raw.size),
                                   scales.ctypes.data_as(C.c_void_p) if scales is not None else None,
                                   C.c_size_t(0 if scales is None else scales.size), 32, C.c_size_t(elems), o.ctypes.data_as(C.c_void_p))
        return o
    g["rwv_int4_down"] = read_weights(4, g["int4_down_packed"], g["int4_down_scales"], g["int4_down_packed"].size * 2)
    g["rwv_int8_down"] = read_weights(3, g["int8_down_w"], g["int8_down_scales"], g["int8_down_w"].size)
    g["rwv_f16_bits"] = allh[::97].copy()
    g["rwv_f16"] = read_weights(1, g["rwv_f16_bits"], None, g["rwv_f16_bits"].size)

    # 8. K-quant tensors through the reference's loader: GGUFLoader::load_tensor (fp32, weight_loader.cpp:520-570 with
    # the block decoders at :125-177) and GGUFLoader::load_tensor_int4 (decode, then the INT4 re-quantiser, :825-957).
    q4k, q6k = kquant_blocks(rng, 12, 8), kquant_blocks(rng, 14, 8)   # 8 super-blocks each: tensors [4 x 512]
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "kq.gguf")
        write_gguf(path,
                   [("llama.embedding_length", 512), ("llama.attention.head_count", 4),
                    ("llama.attention.head_count_kv", 4), ("llama.block_count", 1),
                    ("llama.feed_forward_length", 4), ("llama.context_length", 64)],
                   [("llama.rope.freq_base", 10000.0), ("llama.norm_eps", 1e-5)],
                   [("blk.0.ffn_gate.weight", [4, 512], 12, q4k.tobytes()),
                    ("blk.0.ffn_up.weight", [4, 512], 14, q6k.tobytes())])
        for tag, name, blk in (("q4k", b"blk.0.ffn_gate.weight", q4k), ("q6k", b"blk.0.ffn_up.weight", q6k)):
            f = np.empty(2048, np.float32)
            rc = ref.ref_gguf_load_fp32(path.encode(), name, f.ctypes.data_as(C.c_void_p), C.c_size_t(f.size))
            assert rc == 0, rc
            pk = np.empty(1024, np.uint8)
            sc = np.empty(64, np.float32)
            hs = np.zeros(4, np.float32)
            nh = C.c_uint32(0)
            rc = ref.ref_gguf_load_int4(path.encode(), name, pk.ctypes.data_as(C.c_void_p), C.c_size_t(pk.size),
                                        sc.ctypes.data_as(C.c_void_p), C.c_size_t(sc.size),
                                        hs.ctypes.data_as(C.c_void_p), C.c_size_t(hs.size), C.byref(nh))
            assert rc == 0, rc
            g[tag + "_blocks"], g[tag + "_f32"], g[tag + "_int4_packed"], g[tag + "_int4_scales"] = blk, f, pk, sc

    out = os.path.join(HERE, "ref_golden.npz")
    np.savez_compressed(out, **g)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()

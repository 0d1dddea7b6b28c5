"""ctypes binding of the CPU oracle (oracle/libgreta_oracle.so) and, when it was
built, of the reference's own host code (oracle/_ref/libgreta_ref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of bench.py.  The product package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
FMT_Q4_0, FMT_Q8_0 = 0, 1
ACC_F64, ACC_REF_F32, ACC_FAST_F32 = 0, 1, 2
BLOCK_BYTES = {FMT_Q4_0: 18, FMT_Q8_0: 34}

_lib = None
_ref = None


def build(with_ref=True):
    """Compile the oracle (and oracle/_ref when the reference checkout exists)."""
    target = "all" if with_ref else "libgreta_oracle.so"
    subprocess.run(["make", "-s", "-C", _HERE, target], check=True, stdout=subprocess.DEVNULL)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "libgreta_oracle.so")
        if not os.path.exists(path):
            build(with_ref=False)
        _lib = C.CDLL(path)
        _lib.oracle_fp16_to_fp32.restype = C.c_float
        _lib.oracle_fp16_to_fp32.argtypes = [C.c_uint16]
        _lib.oracle_fp32_to_fp16.restype = C.c_uint16
        _lib.oracle_fp32_to_fp16.argtypes = [C.c_float]
        _lib.oracle_argmax.restype = C.c_int32
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def ref():
    """The reference's own host code, or None when oracle/_ref was not built."""
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libgreta_ref.so")
        if not os.path.exists(path):
            return None
        _ref = C.CDLL(path)
        _ref.ref_half_to_float.restype = C.c_float
        _ref.ref_half_to_float.argtypes = [C.c_uint16]
        _ref.ref_float_to_half.restype = C.c_uint16
        _ref.ref_float_to_half.argtypes = [C.c_float]
    return _ref


def num_threads():
    return lib().oracle_num_threads()


def set_num_threads(n):
    lib().oracle_set_num_threads.argtypes = [C.c_int]
    lib().oracle_set_num_threads.restype = None
    lib().oracle_set_num_threads(int(n))


def set_model_acc(acc):
    """Accumulation used by Model.forward: ACC_F64 (parity, the default) or ACC_FAST_F32 (the timed CPU baseline)."""
    lib().oracle_set_model_acc(C.c_int(acc))


# --------------------------------------------------------------------------- formats
def f16_bits_to_f32(h):
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().oracle_fp16_to_fp32_n(_p(h), _p(out), C.c_size_t(h.size))
    return out


def f32_to_f16_bits(f):
    f = np.ascontiguousarray(f, dtype=np.float32)
    out = np.empty(f.shape, np.uint16)
    lib().oracle_fp32_to_fp16_n(_p(f), _p(out), C.c_size_t(f.size))
    return out


def dequant(blocks, fmt):
    """GGUF blocks (uint8, any shape whose size is a multiple of the block size) -> fp32."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    nb = blocks.size // BLOCK_BYTES[fmt]
    out = np.empty(nb * 32, np.float32)
    lib().oracle_dequant(_p(blocks), C.c_int(fmt), C.c_size_t(nb), _p(out))
    return out


def dequant_ref_int4(packed, scales, group_size=32):
    packed = np.ascontiguousarray(packed, np.uint8)
    scales = np.ascontiguousarray(scales, np.float32)
    out = np.empty(packed.size * 2, np.float32)
    lib().oracle_dequant_ref_int4(_p(packed), _p(scales), C.c_uint32(group_size), C.c_size_t(out.size), _p(out))
    return out


def dequant_ref_int8(w, scales, group_size=32):
    w = np.ascontiguousarray(w, np.int8)
    scales = np.ascontiguousarray(scales, np.float32)
    out = np.empty(w.size, np.float32)
    lib().oracle_dequant_ref_int8(_p(w), _p(scales), C.c_uint32(group_size), C.c_size_t(out.size), _p(out))
    return out


def dequant_q4_k(blocks):
    """Q4_K super-blocks (144 bytes per 256 weights) -> fp32, in the reference's decoding."""
    blocks = np.ascontiguousarray(blocks, np.uint8)
    n = blocks.size // 144
    out = np.empty(n * 256, np.float32)
    lib().oracle_dequant_q4_k(_p(blocks), C.c_size_t(n), _p(out))
    return out


def dequant_q6_k(blocks):
    """Q6_K super-blocks (210 bytes per 256 weights) -> fp32, in the reference's decoding."""
    blocks = np.ascontiguousarray(blocks, np.uint8)
    n = blocks.size // 210
    out = np.empty(n * 256, np.float32)
    lib().oracle_dequant_q6_k(_p(blocks), C.c_size_t(n), _p(out))
    return out


def quantize_q8_0(x):
    """fp32 values (a multiple of 32) -> GGUF Q8_0 blocks."""
    x = np.ascontiguousarray(x, np.float32)
    nb = x.size // 32
    out = np.empty(nb * 34, np.uint8)
    lib().oracle_quantize_q8_0(_p(x), C.c_size_t(nb), _p(out))
    return out


def q4_0_to_ref_int4(blocks):
    blocks = np.ascontiguousarray(blocks, np.uint8)
    nb = blocks.size // 18
    packed = np.empty(nb * 16, np.uint8)
    scales = np.empty(nb, np.float32)
    lib().oracle_q4_0_to_ref_int4(_p(blocks), C.c_size_t(nb), _p(packed), _p(scales))
    return packed, scales


def q8_0_split(blocks):
    blocks = np.ascontiguousarray(blocks, np.uint8)
    nb = blocks.size // 34
    w = np.empty(nb * 32, np.int8)
    scales = np.empty(nb, np.float32)
    lib().oracle_q8_0_split(_p(blocks), C.c_size_t(nb), _p(w), _p(scales))
    return w, scales


def quantize_ref_int4(x):
    x = np.ascontiguousarray(x, np.float32)
    packed = np.zeros((x.size + 1) // 2, np.uint8)
    scales = np.empty((x.size + 31) // 32, np.float32)
    lib().oracle_quantize_ref_int4(_p(x), C.c_size_t(x.size), _p(packed), _p(scales))
    return packed, scales


def quantize_ref_int8(x):
    x = np.ascontiguousarray(x, np.float32)
    w = np.zeros(x.size, np.int8)
    scales = np.empty((x.size + 31) // 32, np.float32)
    lib().oracle_quantize_ref_int8(_p(x), C.c_size_t(x.size), _p(w), _p(scales))
    return w, scales


# --------------------------------------------------------------------------- operators
def gemv(x, w_blocks, fmt, N, K, acc=ACC_F64):
    """x: [M,K] float32 or uint16 (fp16 bits); w_blocks: GGUF blocks of W [N,K]."""
    x = np.ascontiguousarray(x)
    is_f16 = x.dtype == np.uint16
    if not is_f16:
        x = x.astype(np.float32, copy=False)
    M = x.size // K
    w_blocks = np.ascontiguousarray(w_blocks, np.uint8)
    assert w_blocks.size == N * (K // 32) * BLOCK_BYTES[fmt]
    y = np.empty((M, N), np.float32)
    lib().oracle_gemv(_p(x), C.c_int(int(is_f16)), _p(w_blocks), C.c_int(fmt), _p(y), C.c_uint32(M),
                      C.c_uint32(N), C.c_uint32(K), C.c_int(acc))
    return y


def gemm(a, w_blocks, fmt, N, K, out_f16=False, acc=ACC_F64):
    """Prefill form: a [M,K] float32 or uint16 (fp16 bits) -> [M,N] fp32, or fp16 bits."""
    a = np.ascontiguousarray(a)
    is_f16 = a.dtype == np.uint16
    if not is_f16:
        a = a.astype(np.float32, copy=False)
    M = a.size // K
    w_blocks = np.ascontiguousarray(w_blocks, np.uint8)
    assert w_blocks.size == N * (K // 32) * BLOCK_BYTES[fmt]
    c = np.empty((M, N), np.uint16 if out_f16 else np.float32)
    lib().oracle_gemm(_p(a), C.c_int(int(is_f16)), _p(w_blocks), C.c_int(fmt), _p(c), C.c_int(int(out_f16)),
                      C.c_uint32(M), C.c_uint32(N), C.c_uint32(K), C.c_int(acc))
    return c


def gemm_f16w(x, w_bits, N, K, acc=ACC_F64):
    x = np.ascontiguousarray(x, np.float32)
    w_bits = np.ascontiguousarray(w_bits, np.uint16)
    M = x.size // K
    y = np.empty((M, N), np.float32)
    lib().oracle_gemm_f16w(_p(x), _p(w_bits), _p(y), C.c_uint32(M), C.c_uint32(N), C.c_uint32(K), C.c_int(acc))
    return y


def rmsnorm(x, gamma, eps, mode=0):
    x = np.ascontiguousarray(x, np.float32)
    gamma = np.ascontiguousarray(gamma, np.float32)
    cols = gamma.size
    rows = x.size // cols
    y = np.empty_like(x)
    lib().oracle_rmsnorm(_p(x), _p(gamma), _p(y), C.c_uint32(rows), C.c_uint32(cols), C.c_float(eps), C.c_int(mode))
    return y


def rope(x, seq_len, num_heads, head_dim, base, pos_offset):
    y = np.array(x, dtype=np.float32, copy=True, order="C")
    lib().oracle_rope(_p(y), C.c_uint32(seq_len), C.c_uint32(num_heads), C.c_uint32(head_dim), C.c_float(base),
                      C.c_uint32(pos_offset))
    return y


def attention_decode(q, k_cache, v_cache, num_heads, num_heads_kv, head_dim, seq_len, max_seq_len, scale, mode=0):
    """k_cache/v_cache: [Hkv, max_seq, Dh] float32, or uint16 holding fp16 bits."""
    q = np.ascontiguousarray(q, np.float32)
    k_cache = np.ascontiguousarray(k_cache)
    v_cache = np.ascontiguousarray(v_cache)
    is_f16 = k_cache.dtype == np.uint16
    out = np.empty(num_heads * head_dim, np.float32)
    lib().oracle_attention_decode(_p(q), _p(k_cache), _p(v_cache), C.c_int(int(is_f16)), _p(out),
                                  C.c_uint32(num_heads), C.c_uint32(num_heads_kv), C.c_uint32(head_dim),
                                  C.c_uint32(seq_len), C.c_uint32(max_seq_len), C.c_float(scale), C.c_int(mode))
    return out


def attention_prefill(q, k, v, seq_len, num_heads, num_heads_kv, head_dim, scale, causal=True, kv_round_f16=False):
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    o = np.empty(seq_len * num_heads * head_dim, np.float32)
    lib().oracle_attention_prefill(_p(q), _p(k), _p(v), _p(o), C.c_uint32(seq_len), C.c_uint32(num_heads),
                                   C.c_uint32(num_heads_kv), C.c_uint32(head_dim), C.c_float(scale),
                                   C.c_int(int(causal)), C.c_int(int(kv_round_f16)))
    return o.reshape(seq_len, num_heads * head_dim)


def silu_mul(gate, up):
    gate = np.ascontiguousarray(gate, np.float32)
    up = np.ascontiguousarray(up, np.float32)
    y = np.empty_like(gate)
    lib().oracle_silu_mul(_p(gate), _p(up), _p(y), C.c_size_t(gate.size))
    return y


def argmax(logits):
    logits = np.ascontiguousarray(logits, np.float32)
    tie = C.c_int(0)
    i = lib().oracle_argmax(_p(logits), C.c_size_t(logits.size), C.byref(tie))
    return int(i), bool(tie.value)


def embedding(tokens, table_bits, dim, vocab):
    tokens = np.ascontiguousarray(tokens, np.int32)
    table_bits = np.ascontiguousarray(table_bits, np.uint16)
    out = np.empty((tokens.size, dim), np.float32)
    lib().oracle_embedding(_p(tokens), _p(table_bits), _p(out), C.c_uint32(tokens.size), C.c_uint32(dim),
                           C.c_uint32(vocab))
    return out


# --------------------------------------------------------------------------- model
class _Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("wq", "wk", "wv", "wo", "w1", "w2", "w3", "attn_norm", "ffn_norm")]


class _Model(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in
                ("dim", "num_heads", "num_heads_kv", "head_dim", "hidden_dim", "num_layers", "vocab", "max_seq")] + \
               [("rope_base", C.c_float), ("rms_eps", C.c_float), ("fmt", C.c_int), ("layers", C.c_void_p),
                ("tok_embd", C.c_void_p), ("out_norm", C.c_void_p), ("out_weight", C.c_void_p),
                ("k_cache", C.c_void_p), ("v_cache", C.c_void_p)]


class Model:
    """Full-model oracle.  `weights` is the dict produced by the package's
    synthetic-weight generator: per-layer GGUF block arrays and fp32 norms, fp16
    embedding / LM head bits, fp32 output norm."""

    def __init__(self, cfg, weights, fmt=FMT_Q4_0):
        self.cfg = dict(cfg)
        self.keep = weights
        L = cfg["num_layers"]
        self.layers = (_Layer * L)()
        for i, lw in enumerate(weights["layers"]):
            for n in ("wq", "wk", "wv", "wo", "w1", "w2", "w3", "attn_norm", "ffn_norm"):
                setattr(self.layers[i], n, lw[n].ctypes.data)
        n_kv = L * cfg["num_heads_kv"] * cfg["max_seq"] * cfg["head_dim"]
        self.k_cache = np.zeros(n_kv, np.uint16)
        self.v_cache = np.zeros(n_kv, np.uint16)
        m = _Model()
        for n in ("dim", "num_heads", "num_heads_kv", "head_dim", "hidden_dim", "num_layers", "vocab", "max_seq"):
            setattr(m, n, cfg[n])
        m.rope_base, m.rms_eps, m.fmt = cfg["rope_base"], cfg["rms_eps"], fmt
        m.layers = C.cast(self.layers, C.c_void_p)
        m.tok_embd = weights["tok_embd"].ctypes.data
        m.out_norm = weights["out_norm"].ctypes.data
        m.out_weight = weights["out_weight"].ctypes.data
        m.k_cache, m.v_cache = self.k_cache.ctypes.data, self.v_cache.ctypes.data
        self.m = m

    def forward(self, tokens, seq_start):
        tokens = np.ascontiguousarray(tokens, np.int32)
        logits = np.empty(self.cfg["vocab"], np.float32)
        x = np.empty(self.cfg["dim"], np.float32)
        rc = lib().oracle_model_forward(C.byref(self.m), _p(tokens), C.c_uint32(seq_start), C.c_uint32(tokens.size),
                                        _p(logits), _p(x))
        if rc:
            raise ValueError("oracle_model_forward: sequence exceeds max_seq")
        return logits, x

    def generate(self, prompt, n_new):
        """Greedy decoding: returns the n_new generated ids and the top1-top2 logit gap per step."""
        ids, gaps = [], []
        logits, _ = self.forward(prompt, 0)
        pos = len(prompt)
        for _ in range(n_new):
            t, _tie = argmax(logits)
            top2 = np.partition(logits, -2)[-2:]
            gaps.append(float(top2[1] - top2[0]))
            ids.append(t)
            if len(ids) == n_new:
                break
            logits, _ = self.forward(np.array([t], np.int32), pos)
            pos += 1
        return ids, gaps

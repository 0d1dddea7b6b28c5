"""K-quant tensors (GGUF Q4_K / Q6_K): the device decoders against the oracle (which is pinned to the reference's loader),
the re-storing as Q8_0, and a model loaded from a K-quant file."""
import ctypes as C

import numpy as np
import pytest

from _support import load_package, write_gguf
from oracle import oracle as O

GGML_F32, GGML_F16, GGML_Q4_K, GGML_Q6_K = 0, 1, 12, 14
CFG = dict(dim=256, num_heads=4, num_heads_kv=2, num_layers=2, vocab=320, hidden_dim=768, head_dim=64, max_seq=96, rope_base=10000.0, rms_eps=1e-5)


def kquant_blocks(rng, ggml_type, n_super, sigma=0.02):
    """Random super-blocks with super-scales sized so that decoded weights are about N(0, sigma)-sized."""
    if ggml_type == GGML_Q4_K:
        blk = rng.integers(0, 256, (n_super, 144), dtype=np.uint8)
        d = (np.abs(rng.normal(0, sigma, (n_super, 2))) / 256).astype(np.float16)
        blk[:, :4] = d.view(np.uint8).reshape(n_super, 4)
    else:
        blk = rng.integers(0, 256, (n_super, 210), dtype=np.uint8)
        d = (np.abs(rng.normal(0, sigma, n_super)) / 2048).astype(np.float16)
        blk[:, 208:] = d.view(np.uint8).reshape(n_super, 2)
    return blk.reshape(-1)


def decode(blocks, ggml_type):
    return O.dequant_q4_k(blocks) if ggml_type == GGML_Q4_K else O.dequant_q6_k(blocks)


@pytest.fixture(scope="module")
def g():
    pkg = load_package()
    pkg.build()
    pkg.ffi.require_device()
    return pkg.ffi


@pytest.mark.gpu
@pytest.mark.parametrize("ggml_type", [GGML_Q4_K, GGML_Q6_K])
def test_device_decoders_are_the_reference_loaders_bit_for_bit(g, ggml_type):
    rng = np.random.default_rng(70 + ggml_type)
    n_super = 37 * 8
    blk = kquant_blocks(rng, ggml_type, n_super)
    lib = g.cuda()
    assert lib.greta_cuda_kquant_bytes(ggml_type, n_super * 256) == blk.size
    src = g.DeviceBuffer.from_numpy(blk)
    out = g.DeviceBuffer(n_super * 256 * 4)
    g.check(lib.greta_cuda_kquant_dequant(None, ggml_type, src.ptr, n_super * 256, out.ptr, 0))
    want = decode(blk, ggml_type)
    assert np.array_equal(out.download(np.float32).view(np.uint32), want.view(np.uint32))
    half = g.DeviceBuffer(n_super * 256 * 2)
    g.check(lib.greta_cuda_kquant_dequant(None, ggml_type, src.ptr, n_super * 256, half.ptr, 1))
    assert np.array_equal(half.download(np.uint16), O.f32_to_f16_bits(want))
    assert lib.greta_cuda_kquant_dequant(None, 2, src.ptr, 256, out.ptr, 0) != 0             # not a K-quant type
    assert lib.greta_cuda_kquant_dequant(None, ggml_type, src.ptr, 100, out.ptr, 0) != 0     # not whole super-blocks
    for b in (src, out, half):
        b.free()


@pytest.mark.gpu
@pytest.mark.parametrize("ggml_type", [GGML_Q4_K, GGML_Q6_K])
def test_restoring_as_q8_0_gives_the_oracles_blocks_and_a_matching_gemv(g, ggml_type):
    """The planes written by greta_cuda_kquant_to_q8_0 are the oracle's Q8_0 blocks of the decoded values, and the GEMV over
    them stays within the Q8_0 step of the product with the decoded weights themselves."""
    rng = np.random.default_rng(80 + ggml_type)
    N, K = 48, 1024
    blk = kquant_blocks(rng, ggml_type, N * K // 256)
    lib = g.cuda()
    src = g.DeviceBuffer.from_numpy(blk)
    qs = g.DeviceBuffer(lib.greta_cuda_qs_bytes(g.FMT_Q8_0, N, K))
    d = g.DeviceBuffer(lib.greta_cuda_d_bytes(g.FMT_Q8_0, N, K))
    g.check(lib.greta_cuda_kquant_to_q8_0(None, ggml_type, src.ptr, qs.ptr, d.ptr, N, K))
    w = decode(blk, ggml_type)
    want = O.quantize_q8_0(w).reshape(-1, 34)
    assert np.array_equal(qs.download(np.uint8).reshape(-1, 32), want[:, 2:])
    assert np.array_equal(d.download(np.uint16), want[:, :2].copy().view(np.uint16).reshape(-1))      # K / 32 is a multiple of 8: no row padding
    x = rng.normal(0, 1, K).astype(np.float32)
    y = g.DeviceBuffer(N * 4)
    g.check(lib.greta_cuda_gemv(None, g.FMT_Q8_0, g.DeviceBuffer.from_numpy(x).ptr, 0, qs.ptr, d.ptr, y.ptr, 1, N, K))
    got = y.download(np.float32)
    exact_q8 = O.gemv(x, want.reshape(-1), O.FMT_Q8_0, N, K)[0]
    assert np.abs(got - exact_q8).max() <= 2e-5 * np.abs(exact_q8).max()
    exact = w.reshape(N, K).astype(np.float64) @ x.astype(np.float64)
    assert np.abs(got - exact).max() <= 0.01 * np.abs(exact).max() + 1e-6                                # the re-quantisation's own error
    assert lib.greta_cuda_kquant_to_q8_0(None, ggml_type, src.ptr, qs.ptr, d.ptr, N, 96) != 0           # K not whole super-blocks


@pytest.mark.gpu
@pytest.mark.parametrize("ggml_type", [GGML_Q4_K, GGML_Q6_K])
@pytest.mark.parametrize("M,N,K", [(1, 203, 2048), (3, 64, 7168), (1, 1024, 256)])
def test_gemv_straight_from_super_blocks(g, ggml_type, M, N, K):
    """greta_cuda_gemv_kquant reads the weights as they lie in the file (nothing re-quantised): against the product of the
    activations with the oracle's decoded weights in double precision the difference is fp32 rounding."""
    rng = np.random.default_rng(90 + ggml_type + N)
    blk = kquant_blocks(rng, ggml_type, N * K // 256)
    x = rng.normal(0, 1, (M, K)).astype(np.float32)
    lib = g.cuda()
    src, xd = g.DeviceBuffer.from_numpy(blk), g.DeviceBuffer.from_numpy(x)
    y = g.DeviceBuffer(M * N * 4)
    y.fill(0xFF)
    g.check(lib.greta_cuda_gemv_kquant(None, ggml_type, xd.ptr, src.ptr, y.ptr, M, N, K))
    got = y.download(np.float32).reshape(M, N)
    want = x.astype(np.float64) @ decode(blk, ggml_type).reshape(N, K).astype(np.float64).T
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()
    assert lib.greta_cuda_gemv_kquant(None, ggml_type, xd.ptr, src.ptr, y.ptr, M, N, 96) != 0       # K not whole super-blocks
    assert lib.greta_cuda_gemv_kquant(None, ggml_type, xd.ptr, src.ptr, y.ptr, 33, N, K) != 0       # more rows than the route serves
    for b in (src, xd, y):
        b.free()


def _kquant_model_file(path, rng, head):
    """A llama-style file as a Q4_K_M export lays it out: Q4_K projections with Q6_K for ffn_down and attn_v, a Q4_K
    embedding table, and an fp16 or Q6_K LM head.  Returns the oracle's weights: every K-quant tensor decoded and re-stored
    as Q8_0 blocks by the oracle, the embedding decoded and rounded to fp16."""
    D, F, Dh = CFG["dim"], CFG["hidden_dim"], CFG["head_dim"]
    q, kv = CFG["num_heads"] * Dh, CFG["num_heads_kv"] * Dh
    shapes = {"wq": (q, D), "wk": (kv, D), "wv": (kv, D), "wo": (D, q), "w1": (F, D), "w2": (D, F), "w3": (F, D)}
    names = {"wq": "attn_q", "wk": "attn_k", "wv": "attn_v", "wo": "attn_output", "w1": "ffn_gate", "w2": "ffn_down", "w3": "ffn_up"}
    tensors, layers = [], []
    for l in range(CFG["num_layers"]):
        lw = {}
        for n, (r, c) in shapes.items():
            t = GGML_Q6_K if n in ("w2", "wv") else GGML_Q4_K
            blk = kquant_blocks(rng, t, r * c // 256)
            lw[n] = O.quantize_q8_0(decode(blk, t))
            tensors.append((f"blk.{l}.{names[n]}.weight", [r, c], t, blk.tobytes()))
        for n in ("attn_norm", "ffn_norm"):
            lw[n] = rng.normal(1, 0.1, D).astype(np.float32)
            tensors.append((f"blk.{l}.{n}.weight", [D], GGML_F32, lw[n].tobytes()))
        layers.append(lw)
    emb_blk = kquant_blocks(rng, GGML_Q4_K, CFG["vocab"] * D // 256)
    out_norm = rng.normal(1, 0.1, D).astype(np.float32)
    tensors += [("token_embd.weight", [CFG["vocab"], D], GGML_Q4_K, emb_blk.tobytes()), ("output_norm.weight", [D], GGML_F32, out_norm.tobytes())]
    w = {"layers": layers, "tok_embd": O.f32_to_f16_bits(decode(emb_blk, GGML_Q4_K)), "out_norm": out_norm}
    if head == "f16":
        outw = rng.normal(0, 0.02, (CFG["vocab"], D)).astype(np.float16)
        tensors.append(("output.weight", [CFG["vocab"], D], GGML_F16, outw.tobytes()))
        w["out_weight"] = outw.view(np.uint16).reshape(-1)
    else:
        out_blk = kquant_blocks(rng, GGML_Q6_K, CFG["vocab"] * D // 256)
        tensors.append(("output.weight", [CFG["vocab"], D], GGML_Q6_K, out_blk.tobytes()))
        w["out_weight"] = O.quantize_q8_0(decode(out_blk, GGML_Q6_K))
    write_gguf(path,
               [("llama.embedding_length", D), ("llama.attention.head_count", CFG["num_heads"]), ("llama.attention.head_count_kv", CFG["num_heads_kv"]),
                ("llama.block_count", CFG["num_layers"]), ("llama.feed_forward_length", F), ("llama.context_length", CFG["max_seq"])],
               [("llama.rope.freq_base", CFG["rope_base"]), ("llama.norm_eps", CFG["rms_eps"])], tensors)
    return w


def _info(pkg, path):
    from gretacore_v3_b200.model import _Config
    cfg, n = _Config(), C.c_uint32()
    rc = pkg.ffi.host().greta_host_gguf_info(str(path).encode(), C.byref(cfg), C.byref(n))
    return rc, cfg, n.value


def test_parser_maps_kquant_files_to_q8_0_storage(tmp_path):
    pkg = load_package()
    path = tmp_path / "kq.gguf"
    _kquant_model_file(path, np.random.default_rng(4), "q6_k")
    rc, cfg, n = _info(pkg, path)
    assert rc == 0, pkg.ffi.host().greta_host_last_error()
    assert n == CFG["num_layers"] * 9 + 3
    assert cfg.weight_fmt == pkg.ffi.FMT_Q8_0 and cfg.lm_head_fmt == pkg.ffi.FMT_Q8_0
    assert (cfg.dim, cfg.vocab_size, cfg.hidden_dim) == (CFG["dim"], CFG["vocab"], CFG["hidden_dim"])


@pytest.mark.gpu
@pytest.mark.parametrize("head", ["f16", "q6_k"])
def test_model_loaded_from_a_kquant_file(tmp_path, head):
    """A K-quant file generates the ids of the same model whose tensors were decoded and re-stored as Q8_0 by the oracle:
    against the oracle model (fp16 LM head), and against a model handed the oracle's Q8_0 blocks one by one (both heads)."""
    pkg = load_package()
    pkg.build()
    pkg.ffi.require_device()
    path = tmp_path / "kq.gguf"
    weights = _kquant_model_file(path, np.random.default_rng(6), head)
    rc, cfg, _ = _info(pkg, path)
    assert rc == 0
    m = pkg.model.Model(CFG, weight_fmt=cfg.weight_fmt, lm_head_fmt=cfg.lm_head_fmt)
    m.load_gguf(str(path))
    prompt = pkg.model.synth_tokens(5, 20, CFG["vocab"])
    ids, _ = m.generate(prompt, 12)
    m2 = pkg.model.Model(CFG, weight_fmt=pkg.ffi.FMT_Q8_0, lm_head_fmt=cfg.lm_head_fmt)
    m2.load(weights)
    assert m2.generate(prompt, 12)[0] == ids
    if head == "f16":
        want, gaps = O.Model(CFG, weights, O.FMT_Q8_0).generate(prompt, 12)
        assert min(gaps) > 1e-6
        assert ids == want
    m.close()
    m2.close()

"""GGUF file -> device layout: the parser (no device needed) against the reference's own loader where that was built,
and a model loaded from a file against the same model loaded tensor by tensor and against the oracle."""
import ctypes as C
import os

import numpy as np
import pytest

from _support import load_package, q4_0_blocks, q8_0_blocks, write_gguf
from oracle import oracle as O

CFG = dict(dim=256, num_heads=4, num_heads_kv=2, num_layers=2, vocab=320, hidden_dim=768, head_dim=64, max_seq=96, rope_base=10000.0, rms_eps=1e-5)
GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0 = 0, 1, 2, 8


def _model_file(path, fmt_name, rng, tied=False, head="f16"):
    """Writes a llama-style GGUF file of CFG's shape; returns the tensors as the weights dict of the package / oracle."""
    mk, gtype = (q4_0_blocks, GGML_Q4_0) if fmt_name == "q4_0" else (q8_0_blocks, GGML_Q8_0)
    D, F, Dh = CFG["dim"], CFG["hidden_dim"], CFG["head_dim"]
    q, kv = CFG["num_heads"] * Dh, CFG["num_heads_kv"] * Dh
    shapes = {"wq": (q, D), "wk": (kv, D), "wv": (kv, D), "wo": (D, q), "w1": (F, D), "w2": (D, F), "w3": (F, D)}
    names = {"wq": "attn_q", "wk": "attn_k", "wv": "attn_v", "wo": "attn_output", "w1": "ffn_gate", "w2": "ffn_down", "w3": "ffn_up"}
    tensors, layers = [], []
    for l in range(CFG["num_layers"]):
        lw = {}
        for n, (r, c) in shapes.items():
            lw[n] = mk(rng, r, c)
            tensors.append((f"blk.{l}.{names[n]}.weight", [r, c], gtype, lw[n].tobytes()))
        for n, gn in (("attn_norm", "attn_norm"), ("ffn_norm", "ffn_norm")):
            lw[n] = rng.normal(1, 0.1, D).astype(np.float32)
            tensors.append((f"blk.{l}.{gn}.weight", [D], GGML_F32, lw[n].tobytes()))
        layers.append(lw)
    emb = rng.normal(0, 0.02, (CFG["vocab"], D)).astype(np.float16)
    out_norm = rng.normal(1, 0.1, D).astype(np.float32)
    outw = emb if tied else rng.normal(0, 0.02, (CFG["vocab"], D)).astype(np.float16)
    tensors += [("token_embd.weight", [CFG["vocab"], D], GGML_F16, emb.tobytes()), ("output_norm.weight", [D], GGML_F32, out_norm.tobytes())]
    if not tied:
        if head == "f16":
            tensors.append(("output.weight", [CFG["vocab"], D], GGML_F16, outw.tobytes()))
        else:                                   # an fp32 LM head in the file: rounded to fp16 on load
            tensors.append(("output.weight", [CFG["vocab"], D], GGML_F32, outw.astype(np.float32).tobytes()))
    write_gguf(path,
               [("llama.embedding_length", D), ("llama.attention.head_count", CFG["num_heads"]), ("llama.attention.head_count_kv", CFG["num_heads_kv"]),
                ("llama.block_count", CFG["num_layers"]), ("llama.feed_forward_length", F), ("llama.context_length", CFG["max_seq"])],
               [("llama.rope.freq_base", CFG["rope_base"]), ("llama.norm_eps", CFG["rms_eps"])], tensors)
    return {"layers": layers, "tok_embd": emb.view(np.uint16).reshape(-1), "out_norm": out_norm, "out_weight": outw.view(np.uint16).reshape(-1)}


def _info(pkg, path):
    from gretacore_v3_b200.model import _Config
    cfg, n = _Config(), C.c_uint32()
    rc = pkg.ffi.host().greta_host_gguf_info(str(path).encode(), C.byref(cfg), C.byref(n))
    return rc, cfg, n.value


@pytest.mark.parametrize("fmt_name", ["q4_0", "q8_0"])
def test_parser_reads_shape_types_and_tensors(tmp_path, fmt_name):
    pkg = load_package()
    path = tmp_path / "tiny.gguf"
    w = _model_file(path, fmt_name, np.random.default_rng(1))
    rc, cfg, n = _info(pkg, path)
    assert rc == 0, pkg.ffi.host().greta_host_last_error()
    assert n == CFG["num_layers"] * 9 + 3
    assert (cfg.dim, cfg.num_heads, cfg.num_heads_kv, cfg.num_layers, cfg.hidden_dim, cfg.head_dim, cfg.max_seq_len) == \
        (CFG["dim"], CFG["num_heads"], CFG["num_heads_kv"], CFG["num_layers"], CFG["hidden_dim"], CFG["head_dim"], CFG["max_seq"])
    assert cfg.vocab_size == CFG["vocab"]                         # no tokenizer in the file: from the embedding's shape
    assert abs(cfg.rope_base - 10000.0) < 1e-3 and abs(cfg.rms_eps - 1e-5) < 1e-9
    assert cfg.weight_fmt == (pkg.ffi.FMT_Q4_0 if fmt_name == "q4_0" else pkg.ffi.FMT_Q8_0) and cfg.lm_head_fmt == pkg.ffi.FMT_F16
    # the reference's own parser on the same file, where its host code was built (oracle/_ref)
    ref = O.ref()
    if ref is not None:
        got = np.zeros(10, np.uint32)
        assert ref.ref_gguf_config(str(path).encode(), got.ctypes.data_as(C.c_void_p)) == 0
        assert list(got[:4]) == [cfg.dim, cfg.num_heads, cfg.num_heads_kv, cfg.num_layers]
        assert list(got[5:8]) == [cfg.hidden_dim, cfg.head_dim, cfg.max_seq_len]
        assert got[8:10].view(np.float32).tolist() == [np.float32(cfg.rope_base), np.float32(cfg.rms_eps)]
    # a quantised tensor decoded on the host: (float)q * fp32(d), rounded to fp16
    h = pkg.ffi.host()
    name = b"blk.1.ffn_down.weight"
    elems = C.c_size_t()
    assert h.greta_host_gguf_read_fp16(str(path).encode(), name, None, 0, C.byref(elems)) == 0
    assert elems.value == CFG["dim"] * CFG["hidden_dim"]
    out = np.empty(elems.value, np.uint16)
    assert h.greta_host_gguf_read_fp16(str(path).encode(), name, out.ctypes.data, out.size, C.byref(elems)) == 0
    ofmt = O.FMT_Q4_0 if fmt_name == "q4_0" else O.FMT_Q8_0
    assert np.array_equal(out, O.f32_to_f16_bits(O.dequant(w["layers"][1]["w2"], ofmt)))


def test_parser_rejects_what_is_not_a_gguf_file(tmp_path):
    pkg = load_package()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 64)
    assert _info(pkg, bad)[0] != 0 and b"magic" in pkg.ffi.host().greta_host_last_error()
    good = tmp_path / "tiny.gguf"
    _model_file(good, "q4_0", np.random.default_rng(2))
    data = good.read_bytes()
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(data[: len(data) // 2])                     # tensor data reaches past the end
    assert _info(pkg, cut)[0] != 0
    assert _info(pkg, tmp_path / "missing.gguf")[0] != 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt_name,tied,head", [("q4_0", False, "f16"), ("q8_0", True, "f16"), ("q4_0", False, "f32")])
def test_model_loaded_from_a_gguf_file_generates_the_oracle_ids(tmp_path, fmt_name, tied, head):
    pkg = load_package()
    pkg.build()
    pkg.ffi.require_device()
    path = tmp_path / "tiny.gguf"
    weights = _model_file(path, fmt_name, np.random.default_rng(3), tied=tied, head=head)
    rc, cfg, _ = _info(pkg, path)
    assert rc == 0
    m = pkg.model.Model(CFG, weight_fmt=cfg.weight_fmt, lm_head_fmt=cfg.lm_head_fmt)
    m.load_gguf(str(path))
    prompt = pkg.model.synth_tokens(3, 20, CFG["vocab"])
    ids, _ = m.generate(prompt, 12)
    ofmt = O.FMT_Q4_0 if fmt_name == "q4_0" else O.FMT_Q8_0
    want, gaps = O.Model(CFG, weights, ofmt).generate(prompt, 12)
    assert min(gaps) > 1e-6
    assert ids == want
    m2 = pkg.model.Model(CFG, weight_fmt=cfg.weight_fmt, lm_head_fmt=cfg.lm_head_fmt)      # the same tensors, handed over one by one
    m2.load(weights)
    assert m2.generate(prompt, 12)[0] == want
    m.close()
    m2.close()

"""The C++ operator surface that mirrors the reference's (gcore::rt Buffer / GretaArena / graph, gcore::compute
GretaCompute and GretaFused, the launch_* functions with the reference's signatures), driven by a small C++
program (tests/cpp/l1_surface_test.cpp, built by the package's Makefile) on inputs written here, against
expected outputs computed here by the CPU oracle.  Covers the M <= 32 / M > 32 routing of GretaCompute::gemm
for every weight format and the launchers the Python tests do not reach."""
import os
import struct
import subprocess

import numpy as np
import pytest

from _support import ROOT, load_package, q4_0_blocks, q8_0_blocks
from oracle import oracle as O

pytestmark = pytest.mark.gpu
BIN = os.path.join(ROOT, "gretacore-v3_b200", "build", "l1_surface_test")


def _planes(blocks, n_blocks, bb):
    b = blocks.reshape(n_blocks, bb)
    return np.ascontiguousarray(b[:, 2:]).reshape(-1), np.ascontiguousarray(b[:, :2]).reshape(-1)     # payloads, fp16 scales


def _cases():
    rng = np.random.default_rng(123)
    t = {}
    N, K = 256, 512
    nb = N * K // 32
    t["gemm.N"], t["gemm.K"] = np.uint32(N), np.uint32(K)
    b4, b8 = q4_0_blocks(rng, N, K), q8_0_blocks(rng, N, K)
    wf16 = rng.normal(0, 0.02, (N, K)).astype(np.float16)
    t["gemm.q4_0.w"], t["gemm.q4_0.scales"] = _planes(b4, nb, 18)
    t["gemm.q8_0.w"], t["gemm.q8_0.scales"] = _planes(b8, nb, 34)
    t["gemm.int4.w"], t["gemm.int4.scales"] = O.q4_0_to_ref_int4(b4)
    t["gemm.int8.w"], t["gemm.int8.scales"] = O.q8_0_split(b8)
    t["gemm.f16.w"] = wf16.view(np.uint16)
    for M in (1, 32, 33):
        a = rng.normal(0, 1, (M, K)).astype(np.float32)
        t[f"gemm.A{M}"] = a
        for name, blk, fmt in (("q4_0", b4, O.FMT_Q4_0), ("q8_0", b8, O.FMT_Q8_0)):
            t[f"gemm.{name}.want{M}"] = O.gemv(a, blk, fmt, N, K)
            t[f"gemm.{name}.want_tc{M}"] = O.gemm(a, blk, fmt, N, K)         # both operands rounded to fp16, the M > 32 route
        t[f"gemm.int4.want{M}"] = O.gemv(a, b4, O.FMT_Q4_0, N, K)            # the same values in the reference's own storage
        t[f"gemm.int8.want{M}"] = O.gemv(a, b8, O.FMT_Q8_0, N, K)
        t[f"gemm.f16.want{M}"] = O.gemm_f16w(a, wf16.view(np.uint16), N, K)
    import test_kquant as KQ                                                 # weights kept as Q4_K super-blocks (GretaDataType::Q4_K)
    bk = KQ.kquant_blocks(rng, KQ.GGML_Q4_K, N * K // 256)
    t["gemm.q4_k.w"] = bk
    wk = O.dequant_q4_k(bk).reshape(N, K).astype(np.float64)
    for M in (1, 32):
        t[f"gemm.q4_k.want{M}"] = (t[f"gemm.A{M}"].astype(np.float64) @ wk.T).astype(np.float32)
    H, Hkv, Dh, L, S = 8, 2, 64, 200, 256
    q = rng.normal(0, 1, H * Dh).astype(np.float32)
    k = rng.normal(0, 1, (Hkv, S, Dh)).astype(np.float16)
    v = rng.normal(0, 1, (Hkv, S, Dh)).astype(np.float16)
    scale = np.float32(1 / np.sqrt(Dh))
    t["attn.shape"], t["attn.scale"], t["attn.dpos"] = np.array([H, Hkv, Dh, L, S], np.uint32), scale, np.array([L - 1, 0, 0, 0], np.uint32)
    t["attn.q"], t["attn.k16"], t["attn.v16"] = q, k.view(np.uint16), v.view(np.uint16)
    t["attn.k32"], t["attn.v32"] = k.astype(np.float32), v.astype(np.float32)
    t["attn.want"] = O.attention_decode(q, k.view(np.uint16), v.view(np.uint16), H, Hkv, Dh, L, S, float(scale))
    x = rng.normal(0, 1, (5, 320)).astype(np.float32)
    gam = rng.normal(1, 0.1, 320).astype(np.float32)
    t["rms.shape"], t["rms.x"], t["rms.gamma"], t["rms.want"] = np.array([5, 320], np.uint32), x, gam, O.rmsnorm(x, gam, 1e-5)
    D, nq, nkv = 512, 512, 256
    fx = rng.normal(0, 1, D).astype(np.float32)
    fg = rng.normal(1, 0.1, D).astype(np.float32)
    xn = O.rmsnorm(fx.reshape(1, D), fg, 1e-5)
    t["fused.shape"], t["fused.x"], t["fused.gamma"] = np.array([D, nq, nkv], np.uint32), fx, fg
    for name, n in (("wq", nq), ("wk", nkv), ("wv", nkv)):
        blk = q4_0_blocks(rng, n, D)
        t[f"fused.{name}.w"], t[f"fused.{name}.scales"] = _planes(blk, n * D // 32, 18)
        t[f"fused.want_{name[1]}"] = O.gemv(xn, blk, O.FMT_Q4_0, n, D)
    lg = rng.normal(0, 1, 32000).astype(np.float32)
    lg[[777, 20001]] = lg.max() + 1.0                                       # a tie: the first maximum wins
    t["argmax.logits"], t["argmax.want"] = lg, np.uint32(777)
    Hf, Dhf, Sf, pos = 4, 64, 64, 37
    fq = rng.normal(0, 1, Hf * Dhf).astype(np.float32)
    fk = rng.normal(0, 1, (Hf, Sf, Dhf)).astype(np.float32)
    fv = rng.normal(0, 1, (Hf, Sf, Dhf)).astype(np.float32)
    t["frope.shape"], t["frope.scale"], t["frope.dpos"] = np.array([Hf, Dhf, Sf], np.uint32), np.float32(0.125), np.array([pos, 0, 0, 0], np.uint32)
    t["frope.q"], t["frope.k"], t["frope.v"] = fq, fk, fv
    t["frope.want"] = O.attention_decode(O.rope(fq, 1, Hf, Dhf, 10000.0, pos).ravel(), fk, fv, Hf, Hf, Dhf, pos + 1, Sf, 0.125)
    Sp, Hp, Hkvp, Dhp = 70, 4, 2, 64
    pq = rng.normal(0, 1, (Sp, Hp, Dhp)).astype(np.float32)
    pk = rng.normal(0, 1, (Sp, Hkvp, Dhp)).astype(np.float32)
    pv = rng.normal(0, 1, (Sp, Hkvp, Dhp)).astype(np.float32)
    t["prefill.shape"], t["prefill.scale"] = np.array([Sp, Hp, Hkvp, Dhp], np.uint32), np.float32(0.125)
    t["prefill.q"], t["prefill.k"], t["prefill.v"] = pq, pk, pv
    t["prefill.want_causal"] = O.attention_prefill(pq, pk, pv, Sp, Hp, Hkvp, Dhp, 0.125, causal=True)
    t["prefill.want_full"] = O.attention_prefill(pq, pk, pv, Sp, Hp, Hkvp, Dhp, 0.125, causal=False)
    return t


def test_cpp_operator_surface_against_oracle(tmp_path):
    pkg = load_package()
    pkg.build()
    pkg.ffi.require_device()
    res = subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "gretacore-v3_b200", "csrc"), "l1_surface_test"], stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 0 and os.path.exists(BIN), res.stdout[-3000:]
    path = tmp_path / "cases.bin"
    with open(path, "wb") as f:
        for name, arr in _cases().items():
            data = np.ascontiguousarray(arr).tobytes()
            f.write(struct.pack("<I", len(name)) + name.encode() + struct.pack("<Q", len(data)) + data)
    res = subprocess.run([BIN, str(path)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    print(res.stdout)
    assert res.returncode == 0, res.stdout[-4000:]
    assert "0 failed" in res.stdout and res.stdout.count("PASS") >= 45

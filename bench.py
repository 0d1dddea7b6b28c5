#!/usr/bin/env python
"""Benchmark of the quantized-matmul decode path: Llama-2-7B-shaped model, Q4_0 weights, batch 1.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One "step" is one greedy decode step (one token through all 32 layers, the LM head and the
arg-max) after a 512-token random prompt.  The headline numbers printed in one JSON line:
  value      tokens/s with every input resident in HBM (the step is one CUDA-graph launch with the
             next token fed back on the device), timed with CUDA events on the model's stream;
  e2e        the same through the reference-shaped host loop: per step the previous token id goes up
             from pinned host memory and the sampled id comes back before the next step starts;
  roofline   achieved HBM GB/s of the dominant kernel (the fused RMSNorm -> gate/up Q4_0 GEMV ->
             SwiGLU), timed live over the 32 layers' distinct weights (3.6 GB touched per pass, far
             beyond the 126 MB L2), against the measured copy bandwidth of this pool's B200s;
  cpu_baseline  the CPU port of the reference's kernel math (oracle/, OpenMP) on a bounded sample.
With --gpus N > 1 (launched under torchrun, one rank per GPU) the same model runs tensor-parallel: the
weights are sharded Megatron-style, and the exchange after each row-parallel projection is fused into
the GEMV kernels on either side of it over peer memory (--exchange nccl: an all-reduce instead).  Total
work is fixed, so scaling is "strong".

--impl reference times the CPU port itself (the reference ships no CPU implementation of this
path and its GPU kernels are HIP/gfx942 only) on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT_LEN = 512
SEED = 3
METRIC = "decode_tokens_per_s_llama2_7b_shape_q4_0_batch1"


def load_pkg():
    from __graft_entry__ import load_package
    return load_package()


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.rows, self.proc = device, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                                          "-i", str(self.device)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 - 0.05 <= t <= t1 + 0.15 and len(r) >= 9] or [r for _, r in self.rows if len(r) >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[1]) for r in rows)
        reasons = set()
        for r in rows:
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][2]), "reasons": sorted(reasons), "samples": len(rows)}


# ----------------------------------------------------------------------------- CPU baseline (oracle port)
class CpuDecodeSample:
    """The CPU port of the reference's kernel math (oracle/, OpenMP, fp32 accumulation) on a bounded sample of the decode
    workload: ONE whole decode step - embedding, every operator of the layer (norms, the seven quantised projections, RoPE,
    cache write, attention over the cache, SwiGLU, residuals), final norm, LM head - of a 1-layer and of a 2-layer model of
    the workload's shape at the workload's context length.  The difference of the two is the cost of a layer, the rest is
    the per-step fixed cost; a step of the full model is fixed + layers x layer.  The reference has no batch dimension
    (one KV cache, one sequence): a batch of B sequences costs it B steps."""

    def __init__(self, pkg, cfg, context, batch=1):
        from oracle import oracle as O
        self.O, self.cfg, self.batch = O, cfg, batch
        if os.environ.get("TORCHELASTIC_RUN_ID"):        # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU leg runs
            O.set_num_threads(os.cpu_count() or 1)       # on rank 0 alone and may use the whole host
        small = dict(cfg, num_layers=2, max_seq=context + 8)
        weights = pkg.model.synth_weights(small, SEED)
        self.models = []
        for n in (1, 2):
            c = dict(small, num_layers=n)
            w = dict(weights, layers=weights["layers"][:n])
            m = O.Model(c, w)
            m.k_cache[:] = 0x3C00                          # a cache of ones up to the context: the work does not depend on the values
            m.v_cache[:] = 0x3C00
            self.models.append(m)
        self.context = context
        self.tok = np.array([1], np.int32)
        self.cores = O.num_threads()

    def sample(self):
        """One timed decode step of the 1-layer and of the 2-layer model -> (seconds, seconds)."""
        O = self.O
        O.set_model_acc(O.ACC_FAST_F32)
        try:
            t = []
            for m in self.models:
                t0 = time.perf_counter()
                m.forward(self.tok, self.context)
                t.append(time.perf_counter() - t0)
        finally:
            O.set_model_acc(O.ACC_F64)
        return t[0], t[1]

    def step_seconds(self, t1, t2):
        """Seconds the full model's step takes, from the times of the 1-layer and the 2-layer step."""
        layer = max(t2 - t1, 1e-9)
        fixed = max(t1 - layer, 0.0)
        return self.batch * (fixed + self.cfg["num_layers"] * layer)

    def describe(self):
        return (f"one decode step (all operators, context {self.context}) of a 1-layer and a 2-layer model of the workload's shape on the "
                f"CPU port (oracle/greta_oracle.cpp, fp32 accumulation, OpenMP), step = fixed + {self.cfg['num_layers']} x layer"
                + (f", x {self.batch} sequences one after another (the reference has no batch dimension)" if self.batch > 1 else ""))


def cpu_q8_0_gemv_4096(reps=20):
    """The reference's CPU-runnable case: one Q8_0 GEMV, x fp32 [1 x 4096], W [4096 x 4096], seed 0, on the CPU port."""
    from oracle import oracle as O
    rng = np.random.default_rng(0)
    N = K = 4096
    nb = N * (K // 32)
    blk = np.empty((nb, 34), np.uint8)
    blk[:, :2] = (np.abs(rng.normal(0, 0.02, nb)) / 127).astype(np.float16).view(np.uint8).reshape(nb, 2)
    blk[:, 2:] = rng.integers(-127, 128, (nb, 32), dtype=np.int8).view(np.uint8)
    x = rng.normal(0, 1, K).astype(np.float32)
    blk = blk.reshape(-1)
    O.gemv(x, blk, O.FMT_Q8_0, N, K, O.ACC_FAST_F32)
    best = 1e30
    for _ in range(reps):
        t0 = time.perf_counter()
        O.gemv(x, blk, O.FMT_Q8_0, N, K, O.ACC_FAST_F32)
        best = min(best, time.perf_counter() - t0)
    alg = nb * 34 + K * 4 + N * 4
    return {"us": best * 1e6, "gb_per_s": alg / best / 1e9, "algorithmic_bytes": alg, "cores": O.num_threads()}


def cpu_baseline(pkg, cfg, context, batch=1, budget_s=10.0):
    sample = CpuDecodeSample(pkg, cfg, context, batch)
    sample.sample()                                        # warm-up (thread pool, page faults)
    t1s, t2s, t_end = [], [], time.perf_counter() + budget_s
    while len(t1s) < 3 or time.perf_counter() < t_end:
        a, b = sample.sample()
        t1s.append(a)
        t2s.append(b)
    best = sample.step_seconds(float(np.median(t1s)), float(np.median(t2s)))     # medians: a difference of two minima is noise
    return {"value": batch / best, "unit": "tok/s", "cores": sample.cores, "kind": "port",
            "sample": sample.describe() + f"; medians of {len(t1s)} samples in about {budget_s:.0f} s",
            "q8_0_gemv_4096x4096_cpu": cpu_q8_0_gemv_4096()}


def run_reference(args, ranks, cfg, pkg, batch, context):
    """--impl reference: the CPU port of the reference's kernel math on the host cores (rank 0 alone)."""
    if ranks.rank != 0:
        return
    sample = CpuDecodeSample(pkg, cfg, context, batch)
    for _ in range(max(1, min(args.warmup, 3))):
        sample.sample()
    steps = max(1, min(args.steps, 200))
    pairs = [sample.sample() for _ in range(max(steps, 5))]
    ms = 1e3 * sample.step_seconds(float(np.median([p[0] for p in pairs])), float(np.median([p[1] for p in pairs])))
    val = 1e3 * batch / ms
    print(json.dumps({
        "impl": "reference", "metric": metric_name(args), "value": val, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "q4_0 weights, fp32 activations/accumulation", "data": "synthetic",
        "config": dict(workload_config(args, cfg, 1, "host cores"),
                       note="the reference has no CPU implementation of this path and its GPU kernels are HIP/gfx942 only: this arm is "
                            "the CPU port of its kernel math"),
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": sample.cores, "kind": "port",
                         "sample": sample.describe() + f"; medians of {len(pairs)} samples"},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------- roofline of the dominant kernel
def time_dominant_kernel(pkg, cfg, tp, batch=1, reps=4):
    """Fused RMSNorm -> gate/up GEMV -> SwiGLU (single-row or batched form) over distinct weight sets far larger than L2,
    captured in one graph, CUDA events on the launching stream."""
    import ctypes as C
    g = pkg.ffi
    lib = g.cuda()
    D, F = cfg["dim"], cfg["hidden_dim"] // tp
    L = cfg["num_layers"]
    rng = np.random.default_rng(0)
    nb = F * (D // 32)
    qs_h = rng.integers(0, 256, nb * 16, dtype=np.uint8)
    d_h = (np.abs(rng.normal(0, 0.02, nb)) / 8).astype(np.float16).view(np.uint16)
    sets = [(g.DeviceBuffer.from_numpy(qs_h), g.DeviceBuffer.from_numpy(d_h), g.DeviceBuffer.from_numpy(qs_h),
             g.DeviceBuffer.from_numpy(d_h)) for _ in range(max(4, min(L, int(4e9 // (2 * nb * 18)))))]   # >> L2, at most ~4 GB
    x = g.DeviceBuffer.from_numpy(rng.normal(0, 1, batch * D).astype(np.float32))
    gam = g.DeviceBuffer.from_numpy(np.ones(D, np.float32))
    y = g.DeviceBuffer(batch * F * 4)
    ws = g.DeviceBuffer(lib.greta_cuda_gemv_batch_workspace_bytes(batch, D))
    stream = C.c_void_p()
    g.check(lib.greta_cuda_stream_create(C.byref(stream)))

    def one_pass():
        for a, b, c, d in sets:
            if batch == 1:
                g.check(lib.greta_cuda_fused_ffn_front(stream, g.FMT_Q4_0, x.ptr, gam.ptr, 1e-5, a.ptr, b.ptr, c.ptr, d.ptr, y.ptr, D, F))
            else:
                g.check(lib.greta_cuda_fused_ffn_front_batch(stream, g.FMT_Q4_0, x.ptr, gam.ptr, 1e-5, a.ptr, b.ptr, c.ptr, d.ptr, y.ptr, batch, D, F, ws.ptr))

    one_pass()
    g.check(lib.greta_cuda_stream_synchronize(stream))
    graph, ex, e0, e1 = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
    g.check(lib.greta_cuda_graph_capture_begin(stream))
    one_pass()
    g.check(lib.greta_cuda_graph_capture_end(stream, C.byref(graph)))
    g.check(lib.greta_cuda_graph_instantiate(graph, C.byref(ex)))
    lib.greta_cuda_event_create(C.byref(e0))
    lib.greta_cuda_event_create(C.byref(e1))
    for _ in range(3):
        lib.greta_cuda_graph_launch(ex, stream)
    lib.greta_cuda_stream_synchronize(stream)
    lib.greta_cuda_event_record(e0, stream)
    for _ in range(reps):
        lib.greta_cuda_graph_launch(ex, stream)
    lib.greta_cuda_event_record(e1, stream)
    lib.greta_cuda_event_synchronize(e1)
    ms = C.c_float()
    lib.greta_cuda_event_elapsed_ms(e0, e1, C.byref(ms))
    us = ms.value * 1e3 / (reps * len(sets))
    alg_bytes = 2 * nb * 18 + (batch + 1) * D * 4 + batch * F * 4          # both weight matrices + x + gamma in, y out
    for s in sets:
        for b in s:
            b.free()
    name = ("gemv_pipe_kernel<Q4_0, SwiGLU> (fused RMSNorm -> gate/up GEMV -> SwiGLU)" if batch == 1 else
            f"gemv_batch_kernel<Q4_0, SwiGLU> (fused RMSNorm -> gate/up matmul for {batch} rows -> SwiGLU, weights read once)")
    return us, alg_bytes, name


def time_prefill_gemm(pkg, reps=5, split_k=False):
    """The prefill GEMM benchmark shape: fp16 activations [512 x 4096] x Q4_0 weights [11008 x 4096] -> fp16 [512 x 11008] on
    the tcgen05 kernel, 6 distinct weight copies (152 MB, beyond L2) captured in one graph, CUDA events; fraction of the
    measured dense bf16 tensor peak (fp16 runs at the same rate).  split_k: with the tuning switch that lets SMs share a
    tile's K loop (off by default: it changes the fp32 summation order of the prefill)."""
    import ctypes as C
    g = pkg.ffi
    lib = g.cuda()
    g.check(lib.greta_cuda_set_tuning(b"gemm_splitk", 1 if split_k else 0))   # off is the library's default
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, src = float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        peak, src = 1590.0, "fallback"
    M, N, K = 512, 11008, 4096
    rng = np.random.default_rng(1)
    nb = N * (K // 32)
    qs_h = rng.integers(0, 256, nb * 16, dtype=np.uint8)
    d_h = (np.abs(rng.normal(0, 0.02, nb)) / 8).astype(np.float16).view(np.uint16)
    w = [(g.DeviceBuffer.from_numpy(qs_h), g.DeviceBuffer.from_numpy(d_h)) for _ in range(6)]
    a = g.DeviceBuffer.from_numpy(rng.normal(0, 1, (M, K)).astype(np.float16).view(np.uint16))
    c = g.DeviceBuffer(M * N * 2)
    ws = g.DeviceBuffer(lib.greta_cuda_gemm_workspace_bytes(M, K))      # with a workspace the K loop of a tile may be shared between SMs
    stream, graph, ex, e0, e1 = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
    g.check(lib.greta_cuda_stream_create(C.byref(stream)))

    def one_pass():
        for qs, d in w:
            g.check(lib.greta_cuda_gemm(stream, g.FMT_Q4_0, a.ptr, 1, qs.ptr, d.ptr, c.ptr, 1, M, N, K, ws.ptr))

    one_pass()
    g.check(lib.greta_cuda_stream_synchronize(stream))
    g.check(lib.greta_cuda_graph_capture_begin(stream))
    one_pass()
    g.check(lib.greta_cuda_graph_capture_end(stream, C.byref(graph)))
    g.check(lib.greta_cuda_graph_instantiate(graph, C.byref(ex)))
    lib.greta_cuda_event_create(C.byref(e0))
    lib.greta_cuda_event_create(C.byref(e1))
    for _ in range(3):
        lib.greta_cuda_graph_launch(ex, stream)
    lib.greta_cuda_stream_synchronize(stream)
    lib.greta_cuda_event_record(e0, stream)
    for _ in range(reps):
        lib.greta_cuda_graph_launch(ex, stream)
    lib.greta_cuda_event_record(e1, stream)
    lib.greta_cuda_event_synchronize(e1)
    ms = C.c_float()
    lib.greta_cuda_event_elapsed_ms(e0, e1, C.byref(ms))
    us = ms.value * 1e3 / (reps * len(w))
    for qs, d in w:
        qs.free()
        d.free()
    a.free()
    c.free()
    ws.free()
    g.check(lib.greta_cuda_set_tuning(b"gemm_splitk", 0))
    tflops = 2.0 * M * N * K / us / 1e6
    return {"shape": "fp16 [512 x 4096] x Q4_0 [11008 x 4096] -> fp16 [512 x 11008]", "us_per_launch": us, "tflops": tflops, "peak_tflops": peak,
            "frac": tflops / peak, "peak_source": f"of {src}", "bound": "tensor",
            "kernel": "gemm_tc_splitk_kernel (tuning switch gemm_splitk = 1: K loops shared between SMs)" if split_k else "gemm_tc_kernel (default)"}


# ----------------------------------------------------------------------------- GEMV bandwidth per projection shape
def gemv_shapes(pkg):
    """Times the plain Q4_0 / Q8_0 GEMV on every projection shape of the 7B and 70B models (batch 1): distinct weight
    copies totalling ~600 MB rotate so nothing is served from L2, launches are captured in one CUDA graph, CUDA events
    on the launching stream.  Prints one JSON line per shape with GB/s of algorithmic bytes and the fraction of the
    measured HBM peak."""
    import ctypes as C
    g = pkg.ffi
    lib = g.cuda()
    peak, peak_src = measured_peak_gbs()
    stream = C.c_void_p()
    g.check(lib.greta_cuda_stream_create(C.byref(stream)))
    e0, e1 = C.c_void_p(), C.c_void_p()
    lib.greta_cuda_event_create(C.byref(e0))
    lib.greta_cuda_event_create(C.byref(e1))
    rng = np.random.default_rng(0)
    shapes = [("q4_0", g.FMT_Q4_0, n, k) for n, k in [(4096, 4096), (11008, 4096), (4096, 11008), (12288, 4096), (22016, 4096),
                                                      (8192, 8192), (28672, 8192), (8192, 28672)]]
    shapes += [("q8_0", g.FMT_Q8_0, 4096, 4096), ("q8_0", g.FMT_Q8_0, 11008, 4096)]
    for name, fmt, N, K in shapes:
        pb = g.PAYLOAD_BYTES[fmt]
        nb = N * (K // 32)
        wbytes = nb * (pb + 2)
        copies = max(2, int(600e6 // wbytes))
        qs_h = rng.integers(0, 256, nb * pb, dtype=np.uint8)
        d_h = (np.abs(rng.normal(0, 0.02, nb)) / 8).astype(np.float16).view(np.uint16)
        planes = [(g.DeviceBuffer.from_numpy(qs_h), g.DeviceBuffer.from_numpy(d_h)) for _ in range(copies)]
        x = g.DeviceBuffer.from_numpy(rng.normal(0, 1, K).astype(np.float32))
        y = g.DeviceBuffer(N * 4)

        def one_pass():
            for qs, d in planes:
                g.check(lib.greta_cuda_gemv(stream, fmt, x.ptr, 0, qs.ptr, d.ptr, y.ptr, 1, N, K))

        one_pass()
        g.check(lib.greta_cuda_stream_synchronize(stream))
        graph, ex = C.c_void_p(), C.c_void_p()
        g.check(lib.greta_cuda_graph_capture_begin(stream))
        for _ in range(4):
            one_pass()
        g.check(lib.greta_cuda_graph_capture_end(stream, C.byref(graph)))
        g.check(lib.greta_cuda_graph_instantiate(graph, C.byref(ex)))
        lib.greta_cuda_graph_launch(ex, stream)
        lib.greta_cuda_stream_synchronize(stream)
        best = 1e30
        for _ in range(3):
            lib.greta_cuda_event_record(e0, stream)
            lib.greta_cuda_graph_launch(ex, stream)
            lib.greta_cuda_event_record(e1, stream)
            lib.greta_cuda_event_synchronize(e1)
            ms = C.c_float()
            lib.greta_cuda_event_elapsed_ms(e0, e1, C.byref(ms))
            best = min(best, ms.value)
        us = best * 1e3 / (4 * copies)
        alg = wbytes + K * 4 + N * 4
        print(json.dumps({"case": "gemv_shapes", "format": name, "N": N, "K": K, "us_per_launch": round(us, 2),
                          "algorithmic_bytes": alg, "gb_per_s": round(alg / us / 1e3, 1), "frac_of_peak": round(alg / us / 1e3 / peak, 3),
                          "peak_gb_per_s": peak, "peak_source": f"of {peak_src}"}), flush=True)
        lib.greta_cuda_graph_exec_destroy(ex)
        lib.greta_cuda_graph_destroy(graph)
        for qs, d in planes:
            qs.free()
            d.free()
        x.free()
        y.free()


def gemv_batch_shapes(pkg, M=16, prepared=True):
    """Times the batched operators (M activation rows, weights streamed once) on the projection shapes of the 70B and 7B
    models and the grouped-query batched attention at 16 x 4096 keys: distinct weight / cache copies rotate so nothing is
    served from L2, launches are captured in one CUDA graph, CUDA events.  One JSON line per shape."""
    import ctypes as C
    g = pkg.ffi
    lib = g.cuda()
    peak, peak_src = measured_peak_gbs()
    stream = C.c_void_p()
    g.check(lib.greta_cuda_stream_create(C.byref(stream)))
    e0, e1 = C.c_void_p(), C.c_void_p()
    lib.greta_cuda_event_create(C.byref(e0))
    lib.greta_cuda_event_create(C.byref(e1))
    rng = np.random.default_rng(0)

    def timed(one_pass, per_pass):
        one_pass()
        g.check(lib.greta_cuda_stream_synchronize(stream))
        graph, ex = C.c_void_p(), C.c_void_p()
        g.check(lib.greta_cuda_graph_capture_begin(stream))
        for _ in range(3):
            one_pass()
        g.check(lib.greta_cuda_graph_capture_end(stream, C.byref(graph)))
        g.check(lib.greta_cuda_graph_instantiate(graph, C.byref(ex)))
        lib.greta_cuda_graph_launch(ex, stream)
        lib.greta_cuda_stream_synchronize(stream)
        best = 1e30
        for _ in range(3):
            lib.greta_cuda_event_record(e0, stream)
            lib.greta_cuda_graph_launch(ex, stream)
            lib.greta_cuda_event_record(e1, stream)
            lib.greta_cuda_event_synchronize(e1)
            ms = C.c_float()
            lib.greta_cuda_event_elapsed_ms(e0, e1, C.byref(ms))
            best = min(best, ms.value)
        lib.greta_cuda_graph_exec_destroy(ex)
        lib.greta_cuda_graph_destroy(graph)
        return best * 1e3 / (3 * per_pass)

    shapes = [("plain", 8192, 8192), ("plain", 8192, 28672), ("swiglu", 28672, 8192), ("qkv", 10240, 8192), ("plain", 4096, 4096),
              ("swiglu", 11008, 4096), ("plain", 4096, 11008), ("plain", 1024, 8192), ("swiglu", 3584, 8192), ("plain", 8192, 3584)]
    for kind, N, K in shapes:
        rows = 2 * N if kind == "swiglu" else N
        nb = rows * (K // 32)
        wbytes = nb * 18
        copies = max(2, int(700e6 // wbytes))
        qs_h = rng.integers(0, 256, nb * 16, dtype=np.uint8)
        d_h = (np.abs(rng.normal(0, 0.02, nb)) / 8).astype(np.float16).view(np.uint16)
        planes = [(g.DeviceBuffer.from_numpy(qs_h), g.DeviceBuffer.from_numpy(d_h)) for _ in range(copies)]
        x = g.DeviceBuffer.from_numpy(rng.normal(0, 1, M * K).astype(np.float32))
        gam = g.DeviceBuffer.from_numpy(np.ones(K, np.float32))
        y = g.DeviceBuffer(M * rows * 4)
        dpos = g.DeviceBuffer.from_numpy(np.full(M, 7, np.uint32))
        kc = g.DeviceBuffer(M * 8 * 16 * 128 * 2, zero=True)
        ws = g.DeviceBuffer(lib.greta_cuda_gemv_batch_workspace_bytes(M, K)) if prepared else None
        wsp = ws.ptr if ws else None

        def one_pass():
            for qs, d in planes:
                if kind == "plain":
                    g.check(lib.greta_cuda_gemv_batch(stream, g.FMT_Q4_0, x.ptr, None, 0.0, qs.ptr, d.ptr, None, y.ptr, M, N, K, 0, wsp))
                elif kind == "swiglu":
                    half = N * (K // 32)
                    g.check(lib.greta_cuda_fused_ffn_front_batch(stream, g.FMT_Q4_0, x.ptr, gam.ptr, 1e-5, qs.ptr, d.ptr, qs.ptr + half * 16,
                                                                 d.ptr + half * 2, y.ptr, M, K, N, wsp))
                else:                                      # 64 query heads + 8 + 8 KV heads of 128
                    oq, ok = 8192 * (K // 32), 9216 * (K // 32)
                    g.check(lib.greta_cuda_fused_rmsnorm_qkv_rope_kv_batch(stream, g.FMT_Q4_0, x.ptr, gam.ptr, 1e-5, qs.ptr, d.ptr, qs.ptr + oq * 16,
                                                                           d.ptr + oq * 2, qs.ptr + ok * 16, d.ptr + ok * 2, y.ptr, None, None, kc.ptr,
                                                                           kc.ptr, dpos.ptr, M, 64, 8, 128, 16, 500000.0, K, wsp))

        us = timed(one_pass, copies)
        alg = wbytes + M * K * 4 + M * (N if kind != "qkv" else rows) * 4
        print(json.dumps({"case": "gemv_batch_shapes", "op": kind, "prepared_activations": bool(prepared), "rows_of_x": M, "N": N, "K": K, "us_per_launch": round(us, 2),
                          "algorithmic_bytes": alg, "gb_per_s": round(alg / us / 1e3, 1), "frac_of_peak": round(alg / us / 1e3 / peak, 3),
                          "peak_source": f"of {peak_src}"}), flush=True)
        for qs, d in planes:
            qs.free()
            d.free()
        for b in (x, gam, y, dpos, kc):
            b.free()
    # grouped-query batched attention: 16 sequences x 4096 keys, 64 / 8 heads of 128 (and one rank's share under 8-way sharding)
    for H, Hkv in ((64, 8), (8, 1)):
        S, L, Dh = 4160, 4096, 128
        n = M * Hkv * S * Dh
        kv = rng.normal(0, 1, n).astype(np.float16).view(np.uint16)
        copies = max(2, int(600e6 // (2 * n * 2)))
        caches = [(g.DeviceBuffer.from_numpy(kv), g.DeviceBuffer.from_numpy(kv)) for _ in range(copies)]
        q = g.DeviceBuffer.from_numpy(rng.normal(0, 1, M * H * Dh).astype(np.float32))
        o = g.DeviceBuffer(M * H * Dh * 4)
        dpos = g.DeviceBuffer.from_numpy(np.full(M, L - 1, np.uint32))
        nbytes = lib.greta_cuda_attn_decode_scratch_bytes(M * H, Dh)
        scratch = g.DeviceBuffer(nbytes, zero=True)

        def attn_pass():
            for k, v in caches:
                g.check(lib.greta_cuda_attn_decode_batch(stream, q.ptr, k.ptr, v.ptr, o.ptr, dpos.ptr, M, H, Hkv, Dh, S, 0.0884, scratch.ptr, nbytes))

        us = timed(attn_pass, copies)
        alg = 2 * M * Hkv * L * Dh * 2 + 2 * M * H * Dh * 4
        print(json.dumps({"case": "gemv_batch_shapes", "op": "attn_decode_batch", "sequences": M, "heads": H, "kv_heads": Hkv, "keys": L,
                          "us_per_launch": round(us, 2), "algorithmic_bytes": alg, "gb_per_s": round(alg / us / 1e3, 1),
                          "frac_of_peak": round(alg / us / 1e3 / peak, 3), "peak_source": f"of {peak_src}"}), flush=True)
        for k, v in caches:
            k.free()
            v.free()


# ----------------------------------------------------------------------------- small single-kernel cases (for ncu)
def run_case(pkg, name):
    """A few launches of one kernel on a small case whose data is larger than L2, for profiler captures
    (`ncu -k regex:<kernel> ... python bench.py --case <name>`).  Prints nothing but 'ok'."""
    import ctypes as C
    g = pkg.ffi
    g.require_device()
    lib = g.cuda()
    rng = np.random.default_rng(0)

    def planes(N, K, copies):
        nb = N * (K // 32)
        qs = rng.integers(0, 256, nb * 16, dtype=np.uint8)
        d = (np.abs(rng.normal(0, 0.02, nb)) / 8).astype(np.float16).view(np.uint16)
        return [(g.DeviceBuffer.from_numpy(qs), g.DeviceBuffer.from_numpy(d)) for _ in range(copies)]

    if name == "gemv_swiglu":        # 7B FFN front: 50.8 MB per launch, 6 distinct weight sets (305 MB > 126 MB L2)
        D, F = 4096, 11008
        w1, w3 = planes(F, D, 6), planes(F, D, 6)
        x = g.DeviceBuffer.from_numpy(rng.normal(0, 1, D).astype(np.float32))
        gam = g.DeviceBuffer.from_numpy(np.ones(D, np.float32))
        y = g.DeviceBuffer(F * 4)
        for i in range(12):
            a, b = w1[i % 6], w3[i % 6]
            g.check(lib.greta_cuda_fused_ffn_front(None, g.FMT_Q4_0, x.ptr, gam.ptr, 1e-5, a[0].ptr, a[1].ptr, b[0].ptr, b[1].ptr, y.ptr, D, F))
    elif name == "gemv_plain":       # 11008 x 4096 Q4_0 GEMV, 12 distinct copies
        N, K = 11008, 4096
        w = planes(N, K, 12)
        x = g.DeviceBuffer.from_numpy(rng.normal(0, 1, K).astype(np.float32))
        y = g.DeviceBuffer(N * 4)
        for i in range(12):
            g.check(lib.greta_cuda_gemv(None, g.FMT_Q4_0, x.ptr, 0, w[i][0].ptr, w[i][1].ptr, y.ptr, 1, N, K))
    elif name == "gemm_c2":          # the prefill GEMM benchmark shape: 512 x 4096 -> 11008, fp16 in / out
        M, N, K = 512, 11008, 4096
        w = planes(N, K, 6)
        a = g.DeviceBuffer.from_numpy(rng.normal(0, 1, (M, K)).astype(np.float16).view(np.uint16))
        c = g.DeviceBuffer(M * N * 2)
        for i in range(6):
            g.check(lib.greta_cuda_gemm(None, g.FMT_Q4_0, a.ptr, 1, w[i][0].ptr, w[i][1].ptr, c.ptr, 1, M, N, K, None))
    elif name == "gemm_small":       # a prefill chunk of 128 tokens: 128 x 4096 -> 11008, fp16 in / out (dequantisation-bound)
        M, N, K = 128, 11008, 4096
        w = planes(N, K, 6)
        a = g.DeviceBuffer.from_numpy(rng.normal(0, 1, (M, K)).astype(np.float16).view(np.uint16))
        c = g.DeviceBuffer(M * N * 2)
        for i in range(6):
            g.check(lib.greta_cuda_gemm(None, g.FMT_Q4_0, a.ptr, 1, w[i][0].ptr, w[i][1].ptr, c.ptr, 1, M, N, K, None))
    elif name == "attn_decode":      # 32 heads x 128, 2049 keys, fp16 cache, 6 distinct caches (201 MB)
        H, Dh, L, S = 32, 128, 2049, 2304
        kv = rng.normal(0, 1, H * S * Dh).astype(np.float16).view(np.uint16)
        caches = [(g.DeviceBuffer.from_numpy(kv), g.DeviceBuffer.from_numpy(kv)) for _ in range(6)]
        q = g.DeviceBuffer.from_numpy(rng.normal(0, 1, H * Dh).astype(np.float32))
        o = g.DeviceBuffer(H * Dh * 4)
        nbytes = lib.greta_cuda_attn_decode_scratch_bytes(H, Dh)
        scratch = g.DeviceBuffer(nbytes, zero=True)
        for i in range(12):
            k, v = caches[i % 6]
            g.check(lib.greta_cuda_attn_decode(None, q.ptr, k.ptr, v.ptr, o.ptr, None, L, H, H, Dh, S, 0.0884, scratch.ptr, nbytes))
    elif name == "gemv_batch":       # batched plain matmul, 16 rows x (8192 x 8192 Q4_0): 37.7 MB per launch, 5 distinct copies (189 MB)
        M, N, K = 16, 8192, 8192
        w = planes(N, K, 5)
        x = g.DeviceBuffer.from_numpy(rng.normal(0, 1, M * K).astype(np.float32))
        y = g.DeviceBuffer(M * N * 4)
        ws = g.DeviceBuffer(lib.greta_cuda_gemv_batch_workspace_bytes(M, K))
        for i in range(10):
            g.check(lib.greta_cuda_gemv_batch(None, g.FMT_Q4_0, x.ptr, None, 0.0, w[i % 5][0].ptr, w[i % 5][1].ptr, None, y.ptr, M, N, K, 0, ws.ptr))
    elif name == "attn_batch":       # grouped-query batched attention: 16 sequences x 2048 keys, 64 / 8 heads of 128 (134 MB per launch), 2 caches
        M, H, Hkv, Dh, L, S = 16, 64, 8, 128, 2048, 2112
        kv = rng.normal(0, 1, M * Hkv * S * Dh).astype(np.float16).view(np.uint16)
        caches = [(g.DeviceBuffer.from_numpy(kv), g.DeviceBuffer.from_numpy(kv)) for _ in range(2)]
        q = g.DeviceBuffer.from_numpy(rng.normal(0, 1, M * H * Dh).astype(np.float32))
        o = g.DeviceBuffer(M * H * Dh * 4)
        dpos = g.DeviceBuffer.from_numpy(np.full(M, L - 1, np.uint32))
        nbytes = lib.greta_cuda_attn_decode_scratch_bytes(M * H, Dh)
        scratch = g.DeviceBuffer(nbytes, zero=True)
        for i in range(6):
            k, v = caches[i % 2]
            g.check(lib.greta_cuda_attn_decode_batch(None, q.ptr, k.ptr, v.ptr, o.ptr, dpos.ptr, M, H, Hkv, Dh, S, 0.0884, scratch.ptr, nbytes))
    elif name == "decode_step":      # persistent decode-step kernel on a 4-layer model of the 7B shape (0.46 GB of weights)
        from gretacore_v3_b200.model import LLAMA2_7B
        cfg = dict(LLAMA2_7B)
        cfg["num_layers"] = 4
        m = pkg.model.Model(cfg)
        m.load_synthetic(SEED)
        logits = m.forward(pkg.model.synth_tokens(SEED, 512, cfg["vocab"]), 0)
        m.begin_decode(int(np.argmax(logits)), 512)
        m.decode_timed(6)
        m.read_generated(6)
        m.close()
    else:
        raise SystemExit(f"unknown case {name}")
    g.check(lib.greta_cuda_device_synchronize())
    print("ok")


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prompt-len", type=int, default=0, help="prompt tokens per sequence (default 512)")
    ap.add_argument("--batch", type=int, default=0, help="sequences decoding in step (default: 1, or 16 for --workload c5)")
    ap.add_argument("--prefill-chunk", type=int, default=0, help="tokens per prefill call (0 = the whole prompt at once)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", choices=["c4", "c5", "c5-batch1"], default="c4",
                    help="c4: the 7B shape at batch 1 (the metric's workload); c5: the 70B shape at batch 16 (the tensor-parallel scaling "
                         "workload; --prompt-len 4096 --steps 256 for its full size); c5-batch1: the 70B shape at batch 1")
    ap.add_argument("--exchange", choices=["fused", "nccl"], default="fused",
                    help="tensor-parallel exchange of the decode step: fused into the GEMV kernels over peer memory, or NCCL all-reduce")
    ap.add_argument("--case", default=None, help="run a small single-kernel case (gemv_swiglu, gemv_plain, gemm_c2, gemm_small, attn_decode, decode_step, gemv_batch, attn_batch) and exit; "
                         "gemv_shapes prints the GEMV bandwidth of every projection shape")
    args = ap.parse_args()
    pkg = load_pkg()
    ranks = pkg.rendezvous.Ranks()
    if ranks.world != args.gpus and ranks.world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={ranks.world}")

    if args.case == "gemv_shapes":
        pkg.ffi.require_device()
        gemv_shapes(pkg)
        return
    if args.case == "gemv_batch_shapes":
        pkg.ffi.require_device()
        gemv_batch_shapes(pkg, args.batch or 16)
        return
    if args.case:
        run_case(pkg, args.case)
        return
    from gretacore_v3_b200.model import LLAMA2_7B, LLAMA3_70B
    cfg = dict(LLAMA2_7B if args.workload == "c4" else LLAMA3_70B)
    B = args.batch if args.batch else (16 if args.workload == "c5" else 1)
    if args.prompt_len == 0:
        args.prompt_len = PROMPT_LEN
    n_warm = max(args.warmup, 3)
    if args.workload != "c4":                                 # the cache is sized for this run (the 70B shape's full context would be 43 GB at batch 16)
        cfg["max_seq"] = (args.prompt_len + n_warm + args.steps + 8 + 63) // 64 * 64
    if args.prompt_len + n_warm + args.steps > cfg["max_seq"]:
        raise SystemExit(f"prompt {args.prompt_len} + warm-up {n_warm} + steps {args.steps} exceed the cache of {cfg['max_seq']} positions")
    context = args.prompt_len + n_warm + args.steps // 2
    if args.impl == "reference":
        run_reference(args, ranks, cfg, pkg, B, context)
        return

    import ctypes as C
    g = pkg.ffi
    g.require_device()                       # raises when the CUDA library or a device is missing: no CPU fallback
    lib = g.cuda()
    g.check(lib.greta_cuda_set_device(ranks.local))
    tp = ranks.world
    model = pkg.model.Model(cfg, tp_rank=ranks.rank, tp_size=tp, batch=B)
    if tp > 1:
        uid = (C.c_char * 128)()
        if ranks.rank == 0:
            g.check(lib.greta_cuda_comm_unique_id(uid))
        raw = ranks.bcast(bytes(uid.raw), 128)
        comm = C.c_void_p()
        idbuf = C.create_string_buffer(raw, 128)
        g.check(lib.greta_cuda_comm_init(C.byref(comm), idbuf, tp, ranks.rank), "comm_init")
        model.set_comm(comm)
        if args.exchange == "fused":
            peer_keep = pkg.rendezvous.install_peer_exchange(model, ranks, cfg["dim"], batch=B)
            if peer_keep is None:
                args.exchange = "nccl (peer memory could not be mapped)"
            elif B > 1:
                args.exchange = "all-reduce over peer memory (one kernel per rank)"
    model.load_synthetic(SEED if args.workload == "c4" else 4)
    seed = SEED if args.workload == "c4" else 4
    prompts = [pkg.model.synth_tokens(seed, args.prompt_len, cfg["vocab"], stream=(1 << 40) + b) for b in range(B)]
    chunk = args.prefill_chunk or args.prompt_len           # prefill (not timed): one tensor-core pass per sequence by default
    first = []
    for b in range(B):
        if B > 1:
            model.set_sequence(b)
        for c0 in range(0, args.prompt_len, chunk):
            logits = model.forward(prompts[b][c0:c0 + chunk], c0)
        first.append(int(np.argmax(logits)))
    pos = args.prompt_len
    first_arg = first[0] if B == 1 else first

    # ---- value: device-resident decode loop, CUDA events, max over ranks
    model.begin_decode(first_arg, pos)
    model.decode_timed(n_warm)
    sampler = ClockSampler(ranks.local)
    if ranks.rank == 0:
        sampler.start()
        time.sleep(0.3)
    ranks.barrier()
    g.check(lib.greta_cuda_device_synchronize())
    launches0 = lib.greta_cuda_launch_count()
    t0 = time.time()
    ms = model.decode_timed(args.steps)
    g.check(lib.greta_cuda_device_synchronize())
    launches = lib.greta_cuda_launch_count() - launches0
    ms = ranks.gather_max(float(ms))
    ids_dev = np.asarray(model.read_generated(n_warm + args.steps)).reshape(B, -1)

    # ---- e2e: host-driven loop (token ids up, sampled ids down, every step), restarted from the same state
    ranks.barrier()
    model.decode_e2e(first_arg, pos, n_warm)                                 # warm-up of this loop
    ids_e2e, ms_e2e = model.decode_e2e(first_arg, pos, args.steps)
    ids_e2e = np.asarray(ids_e2e).reshape(B, -1)
    ms_e2e = ranks.gather_max(float(ms_e2e))
    clocks = sampler.stop(t0, time.time()) if ranks.rank == 0 else None      # sampled over both timed loops
    same = bool(np.array_equal(ids_e2e, ids_dev[:, :args.steps]))
    oracle_check = check_against_stored_oracle_ids(args, cfg, prompts[0], [first[0]] + ids_dev[0].tolist(), [first[0]] + ids_e2e[0].tolist())

    if ranks.rank != 0:
        return
    # ---- roofline of the dominant kernel and the CPU baseline (rank 0)
    model.close()
    us, alg, kernel_name = time_dominant_kernel(pkg, cfg, tp, B)
    peak, peak_src = measured_peak_gbs()
    achieved = alg / us / 1e3
    roofline = {"bound": "hbm", "kernel": kernel_name,
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": f"of {peak_src}",
                "us_per_launch": us, "algorithmic_bytes_per_launch": alg,
                # dram__bytes_read + write per launch, from the ncu capture of the 7B-sized single-row kernel (50.83 MB for
                # 50.80 MB algorithmic; summary under profiles/), scaled by the bytes this launch moves
                "traffic": int(alg * 50830848 / 50801664)}
    tok_s = 1e3 * B * args.steps / ms
    # whole-step view of the same bound: bytes one decode step must read
    step_bytes = model_step_bytes(cfg, pos + n_warm + args.steps // 2, B)
    out = {
        "metric": metric_name(args),
        "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": ("q4_0 weights (int8 dot products on 23-bit fixed-point activations), fp32 accumulation, fp16 KV cache" if B == 1 else
                  "q4_0 weights (exact integer weights x activations as fp16 pairs on the tensor cores), fp32 accumulation, fp16 KV cache"),
        "data": "synthetic",
        "config": workload_config(args, cfg, tp, f"tp{tp}, exchange {args.exchange}" if tp > 1 else "single GPU", B),
        "clocks": clocks, "gpu_launches": int(launches),
        "e2e": {"value": 1e3 * B * args.steps / ms_e2e, "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
                "ids_match_device_loop": same},
        "ids_match_oracle": oracle_check["match"], "ids_checked": oracle_check,
        "roofline": roofline,
        "step_hbm": {"bytes_per_step": step_bytes, "achieved_gbs": step_bytes / (ms / args.steps) / 1e6,
                     "frac_of_peak": step_bytes / (ms / args.steps) / 1e6 / (peak * tp),
                     "note": "aggregate over the N GPUs; the fraction is of N x the measured per-GPU peak"},
    }
    if tp == 1:                                              # reported at N=1 only
        out["prefill_gemm"] = time_prefill_gemm(pkg)         # the tensor-bound half of the path: the prefill dequant-GEMM
        out["prefill_gemm_split_k"] = time_prefill_gemm(pkg, split_k=True)   # the same product with the opt-in split over K
    if not args.no_cpu_baseline and tp == 1:
        out["cpu_baseline"] = cpu_baseline(pkg, cfg, context, B)
    print(json.dumps(out))


def metric_name(args):
    if args.workload == "c4":
        return METRIC if (args.batch or 1) == 1 else f"decode_tokens_per_s_llama2_7b_shape_q4_0_batch{args.batch}"
    return f"decode_tokens_per_s_llama3_70b_shape_q4_0_batch{args.batch or (16 if args.workload == 'c5' else 1)}"


def workload_config(args, cfg, tp, parallelism, batch=1):
    shape = (f"{cfg['num_layers']} layers, hidden {cfg['dim']}, {cfg['num_heads']}/{cfg['num_heads_kv']} heads x {cfg['head_dim']}, "
             f"FFN {cfg['hidden_dim']}, vocab {cfg['vocab']}")
    name = "Llama-2-7B-shaped" if args.workload == "c4" else "Llama-3-70B-shaped"
    return {"workload": f"{name} model ({shape}), random-init Q4_0 weights, fp16 LM head, {args.prompt_len}-token random prompt then greedy "
                        f"decode at batch {batch}" + (" (every sequence its own prompt, cache and position)" if batch > 1 else ""),
            "prompt_len": args.prompt_len, "parallelism": parallelism,
            "batch": batch,
            "l2_defeat": f"every step streams {model_step_bytes(cfg, args.prompt_len, batch) / 1e9:.1f} GB of distinct weights and cache (L2 is 126 MB)",
            "seed": SEED}


def check_against_stored_oracle_ids(args, cfg, prompt, ids_device_loop, ids_host_loop):
    """Compares the ids of the timed runs with the CPU oracle's ids for the same seeded workload, stored in
    tests/golden/model_ids.npz (the oracle needs minutes of host time for them; tests/golden/make_model_ids.py wrote
    them).  Only the default workload (7B shape, seed 3, 512-token prompt) has stored ids; `match` is None otherwise."""
    path = os.path.join(ROOT, "tests", "golden", "model_ids.npz")
    name = "llama2_7b_seed3"
    if args.workload != "c4" or not os.path.exists(path):
        return {"match": None, "why": "no stored oracle ids for this workload"}
    gold = np.load(path)
    want, wprompt = gold[name + ".ids"][0].tolist(), gold[name + ".prompts"][0]
    if len(prompt) != len(wprompt) or not np.array_equal(prompt, wprompt):
        return {"match": None, "why": "prompt differs from the stored workload's"}
    n_dev, n_host = min(len(want), len(ids_device_loop)), min(len(want), len(ids_host_loop))
    ok = ids_device_loop[:n_dev] == want[:n_dev] and ids_host_loop[:n_host] == want[:n_host]
    return {"match": bool(ok), "device_loop_ids_compared": n_dev, "host_loop_ids_compared": n_host,
            "oracle_min_top2_gap": float(gold[name + ".gaps"][0].min())}


def model_step_bytes(cfg, pos, batch=1):
    """Bytes one decode step must read: the weights once, and every sequence's keys and values."""
    D, F, L, V = cfg["dim"], cfg["hidden_dim"], cfg["num_layers"], cfg["vocab"]
    kv = cfg["num_heads_kv"] * cfg["head_dim"]
    w = L * ((2 * D * D + 2 * D * kv + 3 * D * F) * 18 // 32)
    return w + V * D * 2 + batch * L * 2 * kv * 2 * (pos + 1)


if __name__ == "__main__":
    main()

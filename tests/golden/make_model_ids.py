"""Generates tests/golden/model_ids.npz: greedy ids of the CPU oracle on the full-size model workloads.

The oracle (oracle/greta_oracle.cpp) needs minutes of host CPU time for a 32-layer model with a 512-token prompt,
too long for a test run; its output on the seeded workload is therefore stored once and the GPU tests and
bench.py compare against the stored ids.  The inputs are the package's counter-based synthetic tensors
(libgreta_host.so; no GPU needed to generate them), so the same seed gives the same bytes everywhere.

    python tests/golden/make_model_ids.py [case ...]        # default: every case

Cases:
  llama2_7b_seed3   32 layers, hidden 4096, 32 heads x 128, FFN 11008, vocab 32000, Q4_0, fp16 LM head; 512 random
                    prompt ids, 128 greedy steps, seed 3 (the workload of the decode tokens/s metric).
  llama3_70b_l2_seed4_b16
                    the 70B shape (hidden 8192, GQA 64/8 x 128, FFN 28672, vocab 128256, rope 500000) cut to 2 layers,
                    16 sequences with their own 48-token random prompts, 8 greedy steps each, seed 4 (the batched
                    tensor-parallel workload at a layer count the oracle can run).
Stored per case: ids [B][n_new], top-2 logit gap per step [B][n_new], prompts [B][prompt_len], seed, and the shape.
"""
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from _support import load_package  # noqa: E402
from oracle import oracle as O  # noqa: E402

OUT = os.path.join(HERE, "model_ids.npz")


def cases(pkg):
    from gretacore_v3_b200.model import LLAMA2_7B, LLAMA3_70B
    c70 = dict(LLAMA3_70B)
    c70["num_layers"] = 2
    c70["max_seq"] = 64
    return {
        "llama2_7b_seed3": dict(cfg=dict(LLAMA2_7B), seed=3, batch=1, prompt_len=512, n_new=128),
        "llama3_70b_l2_seed4_b16": dict(cfg=c70, seed=4, batch=16, prompt_len=48, n_new=8),
    }


def prompt_of(pkg, seed, b, n, vocab):
    """Sequence b of a batch draws its prompt from its own stream of the generator (sequence 0 = the batch-1 prompt)."""
    return pkg.model.synth_tokens(seed, n, vocab, stream=(1 << 40) + b)


def run_case(pkg, name, c):
    cfg, seed = c["cfg"], c["seed"]
    t0 = time.time()
    weights = pkg.model.synth_weights(cfg, seed)
    ids, gaps, prompts = [], [], []
    for b in range(c["batch"]):
        prompt = prompt_of(pkg, seed, b, c["prompt_len"], cfg["vocab"])
        i, g = O.Model(cfg, weights).generate(prompt, c["n_new"])
        ids.append(i)
        gaps.append(g)
        prompts.append(prompt)
        print(f"{name}: sequence {b} done after {time.time() - t0:.0f} s, smallest gap {min(g):.3e}", flush=True)
    return {f"{name}.ids": np.array(ids, np.int32), f"{name}.gaps": np.array(gaps, np.float64),
            f"{name}.prompts": np.array(prompts, np.int32), f"{name}.seed": np.int64(seed),
            f"{name}.shape": np.array([cfg[k] for k in ("dim", "num_heads", "num_heads_kv", "num_layers", "vocab", "hidden_dim",
                                                        "head_dim", "max_seq")], np.int64)}


def main():
    pkg = load_package()
    O.set_num_threads(os.cpu_count() or 1)
    todo = cases(pkg)
    want = sys.argv[1:] or list(todo)
    store = dict(np.load(OUT)) if os.path.exists(OUT) else {}
    for name in want:
        store.update(run_case(pkg, name, todo[name]))
        np.savez_compressed(OUT, **store)
    print("wrote", OUT, sorted(store))


if __name__ == "__main__":
    main()

"""Full-size greedy-token parity on the metric's own workload: the Llama-2-7B-shaped model, 512-token prompt
(prefilled through the tensor-core GEMM), then greedy decode steps on the device loop, against the CPU oracle
running the same seeded weights.  Minutes of host CPU time and ~8 GB of host memory: runs only with
GRETA_FULL_PARITY=1 (and GRETA_FULL_PARITY_STEPS to change the number of decode steps, default 128)."""
import os
import time

import numpy as np
import pytest

from _support import load_package
from oracle import oracle as O

pytestmark = [pytest.mark.gpu, pytest.mark.slow]


@pytest.mark.skipif(os.environ.get("GRETA_FULL_PARITY") != "1", reason="set GRETA_FULL_PARITY=1 (minutes of CPU time)")
def test_7b_shape_greedy_ids_match_oracle():
    pkg = load_package()
    pkg.build()
    pkg.ffi.require_device()
    from gretacore_v3_b200.model import LLAMA2_7B
    cfg, seed = dict(LLAMA2_7B), 3
    n_new = int(os.environ.get("GRETA_FULL_PARITY_STEPS", "128"))
    prompt = pkg.model.synth_tokens(seed, 512, cfg["vocab"])
    m = pkg.model.Model(cfg)
    m.load_synthetic(seed)
    t0 = time.time()
    ids, _ = m.generate(prompt, n_new)
    m.close()
    t1 = time.time()
    O.set_num_threads(os.cpu_count() or 1)
    weights = pkg.model.synth_weights(cfg, seed)
    want, gaps = O.Model(cfg, weights).generate(prompt, n_new)
    t2 = time.time()
    first_diff = next((i for i, (a, b) in enumerate(zip(ids, want)) if a != b), None)
    print(f"GPU {t1 - t0:.1f} s, oracle {t2 - t1:.1f} s, smallest top-2 logit gap {min(gaps):.3e}, first difference {first_diff}")
    assert ids == want, (first_diff, ids[:8], want[:8])

"""Tensor parallelism on real GPUs: 2 ranks (one process per GPU, NCCL) give the oracle's greedy ids.
Skipped when fewer than two devices are visible."""
import json
import os
import subprocess
import sys

import pytest

from _support import ROOT, load_package

pytestmark = pytest.mark.gpu


def test_two_rank_tensor_parallel_decode_matches_oracle():
    pkg = load_package()
    pkg.build()
    if pkg.ffi.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(ROOT, "tests", "_tp_worker.py")]
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    lines = [l for l in res.stdout.splitlines() if l.startswith("TP_RESULT ")]
    assert res.returncode == 0 and lines, res.stdout[-3000:]
    out = json.loads(lines[-1][len("TP_RESULT "):])
    assert out["ok"], out

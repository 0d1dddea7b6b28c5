"""One rank of the tensor-parallel check (launched by test_tp_gpu.py under torch.distributed.run).
Each rank holds its shard of a small Llama-shaped model, runs prefill + greedy decode with the NCCL
exchange installed, and rank 0 compares the ids with the CPU oracle's."""
import ctypes as C
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from _support import load_package  # noqa: E402
import bench  # noqa: E402

CFG = dict(dim=512, num_heads=8, num_heads_kv=4, num_layers=3, vocab=2048, hidden_dim=1536, head_dim=64, max_seq=96,
           rope_base=10000.0, rms_eps=1e-5)


def main():
    ranks = bench.Ranks()
    pkg = load_package()
    g = pkg.ffi
    lib = g.cuda()
    g.check(lib.greta_cuda_set_device(ranks.local))
    uid = (C.c_char * 128)()
    if ranks.rank == 0:
        g.check(lib.greta_cuda_comm_unique_id(uid))
    raw = ranks.bcast(bytes(uid.raw), 128)
    comm = C.c_void_p()
    g.check(lib.greta_cuda_comm_init(C.byref(comm), C.create_string_buffer(raw, 128), ranks.world, ranks.rank), "comm_init")
    seed, n_new = 9, 16
    m = pkg.model.Model(CFG, tp_rank=ranks.rank, tp_size=ranks.world)
    m.set_comm(comm)
    m.load_synthetic(seed)
    out = {}
    for plen in (12, 40):                       # GEMV-route prefill and tensor-core prefill
        prompt = pkg.model.synth_tokens(seed, plen, CFG["vocab"])
        ids, _ = m.generate(prompt, n_new)
        out[str(plen)] = ids
    ranks.barrier()
    if ranks.rank == 0:
        from oracle import oracle as O
        weights = pkg.model.synth_weights(CFG, seed)
        ok = True
        for plen in (12, 40):
            prompt = pkg.model.synth_tokens(seed, plen, CFG["vocab"])
            want, gaps = O.Model(CFG, weights).generate(prompt, n_new)
            ok = ok and out[str(plen)] == want and min(gaps) > 1e-6
            out["want" + str(plen)] = want
        out["ok"] = bool(ok)
        print("TP_RESULT " + json.dumps(out), flush=True)
    m.close()
    g.check(lib.greta_cuda_comm_destroy(comm))


if __name__ == "__main__":
    main()

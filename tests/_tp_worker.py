"""One rank of the tensor-parallel check (launched by test_tp_gpu.py under torch.distributed.run).
Each rank holds its shard of a small Llama-shaped model and runs prefill + greedy decode twice: with the NCCL
all-reduce, and with the exchange fused into the GEMV kernels over peer memory; then a batch of five sequences
decoding in step (NCCL all-reduce, then the all-reduce through peer memory), then a model loaded from a K-quant file; rank 0 compares all ids with the CPU oracle's and reads the
exchange's time-out status."""
import ctypes as C
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from _support import load_package  # noqa: E402

CFG = dict(dim=512, num_heads=8, num_heads_kv=4, num_layers=3, vocab=2048, hidden_dim=1536, head_dim=64, max_seq=96,
           rope_base=10000.0, rms_eps=1e-5)


def main():
    pkg = load_package()
    ranks = pkg.rendezvous.Ranks()
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
    out = {}
    for mode in ("nccl", "fused"):
        m = pkg.model.Model(CFG, tp_rank=ranks.rank, tp_size=ranks.world)
        m.set_comm(comm)
        keep = pkg.rendezvous.install_peer_exchange(m, ranks, CFG["dim"]) if mode == "fused" else None
        m.load_synthetic(seed)
        for plen in (12, 40, 12):               # GEMV-route prefill, tensor-core prefill, and a session that restarts earlier
            prompt = pkg.model.synth_tokens(seed, plen, CFG["vocab"])
            ids, _ = m.generate(prompt, n_new)
            if out.setdefault(mode + str(plen), ids) != ids:
                out["repeat_mismatch"] = True
        ranks.barrier()
        m.close()
        if mode == "fused" and keep is None:
            out["peer_setup_failed"] = True
        if keep:
            code = C.c_int(-1)
            g.check(lib.greta_cuda_peer_status(C.byref(code)))
            out["peer_status"] = code.value
            for ptr in keep[2]:
                g.check(lib.greta_cuda_ipc_close(ptr))
            ranks.barrier()
            keep[0].free()
    # a batch of sequences under tensor parallelism (batched kernels, all-reduce over [batch x dim], logits gathered per rank slice)
    B, blen = 5, 14
    bprompts = np.stack([pkg.model.synth_tokens(seed, blen, CFG["vocab"], stream=(1 << 40) + b) for b in range(B)])
    for mode in ("batch", "batch_peer"):           # NCCL all-reduce, then the all-reduce through peer memory
        m = pkg.model.Model(CFG, tp_rank=ranks.rank, tp_size=ranks.world, batch=B)
        m.set_comm(comm)
        keep = pkg.rendezvous.install_peer_exchange(m, ranks, CFG["dim"], batch=B) if mode == "batch_peer" else None
        m.load_synthetic(seed)
        out[mode] = m.generate_batch(bprompts, n_new).tolist()
        out[mode + "_again"] = m.generate_batch(bprompts, n_new).tolist()      # a second session restarts at the earlier positions
        ranks.barrier()
        m.close()
        if mode == "batch_peer" and keep is None:
            out["peer_setup_failed"] = True
        if keep:
            code = C.c_int(-1)
            g.check(lib.greta_cuda_peer_status(C.byref(code)))
            out["peer_status_batch"] = code.value
            for ptr in keep[2]:
                g.check(lib.greta_cuda_ipc_close(ptr))
            ranks.barrier()
            keep[0].free()
    # a K-quant file under tensor parallelism: every rank decodes its rows on the device, re-stores them as Q8_0 and keeps its
    # column range (the down-projection's 384 columns per rank are not whole super-blocks)
    import tempfile
    import test_kquant as KQ
    with tempfile.TemporaryDirectory() as td:
        kpath = os.path.join(td, "kq.gguf")
        kweights = KQ._kquant_model_file(kpath, np.random.default_rng(6), "f16")        # the same file on every rank
        m = pkg.model.Model(KQ.CFG, tp_rank=ranks.rank, tp_size=ranks.world, weight_fmt=g.FMT_Q8_0)
        m.set_comm(comm)
        m.load_gguf(kpath)
        kprompt = pkg.model.synth_tokens(5, 20, KQ.CFG["vocab"])
        out["kquant"] = m.generate(kprompt, 12)[0]
        ranks.barrier()
        m.close()
    if ranks.rank == 0:
        from oracle import oracle as O
        want, gaps = O.Model(KQ.CFG, kweights, O.FMT_Q8_0).generate(kprompt, 12)
        out["kquant_ok"] = out["kquant"] == want and min(gaps) > 1e-6
        weights = pkg.model.synth_weights(CFG, seed)
        ok = True
        for plen in (12, 40):
            prompt = pkg.model.synth_tokens(seed, plen, CFG["vocab"])
            want, gaps = O.Model(CFG, weights).generate(prompt, n_new)
            ok = ok and out["nccl" + str(plen)] == want and out["fused" + str(plen)] == want and min(gaps) > 1e-6
            out["want" + str(plen)] = want
        for b in range(B):
            want, gaps = O.Model(CFG, weights).generate(bprompts[b], n_new)
            ok = ok and min(gaps) > 1e-6 and all(out[k][b] == want for k in ("batch", "batch_again", "batch_peer", "batch_peer_again"))
        out["ok"] = (bool(ok) and out.get("peer_status") == 0 and out.get("peer_status_batch") == 0 and not out.get("repeat_mismatch")
                     and not out.get("peer_setup_failed") and out["kquant_ok"])
        print("TP_RESULT " + json.dumps(out), flush=True)
    g.check(lib.greta_cuda_comm_destroy(comm))


if __name__ == "__main__":
    main()

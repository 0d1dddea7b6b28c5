"""Host-side logic of the multi-GPU path, on CPU with two processes: the package's rendezvous star
(hand-out of the NCCL id, gathering of timings), and the tensor-parallel algebra (row-split
and column-split shards from the host layer's tensor_shard, partial products summed across ranks)
checked with the CPU oracle standing in for the kernels."""
import ctypes as C
import multiprocessing as mp
import os
import struct

import numpy as np

from _support import ROOT, load_package, q4_0_blocks

CFG = dict(dim=256, num_heads=4, num_heads_kv=2, hidden_dim=768, head_dim=64)


def _shard(pkg, which, rank, world):
    from gretacore_v3_b200.model import _Config
    c = _Config(CFG["dim"], CFG["num_heads"], CFG["num_heads_kv"], 1, 1000, CFG["hidden_dim"], CFG["head_dim"], 64, 1e4, 1e-5,
                pkg.ffi.FMT_Q4_0, pkg.ffi.FMT_F16, rank, world)
    out = (C.c_uint32 * 6)()
    assert pkg.ffi.host().greta_host_tensor_shard(C.byref(c), which, out) == 0
    return list(out)


def _rank_main(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import sys
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle import oracle as O
    pkg = load_package()
    ranks = pkg.rendezvous.Ranks()
    # 1. id hand-out: every rank ends up with rank 0's 128 bytes
    uid = bytes(range(128)) if rank == 0 else b"\0" * 128
    got = ranks.bcast(uid, 128)
    ranks.barrier()
    # 2. max over ranks lands on rank 0; the all-gather that swaps the exchange buffers' IPC handles
    mx = ranks.gather_max(10.0 + rank)
    handles = ranks.allgather(bytes([rank + 1]) * 64)
    assert handles == [bytes([r + 1]) * 64 for r in range(world)]
    # 3. column-parallel gate (rows split) then row-parallel down (K split), partial sums exchanged through rank 0
    rng = np.random.default_rng(5)
    D, F = CFG["dim"], CFG["hidden_dim"]
    w1, w2 = q4_0_blocks(rng, F, D), q4_0_blocks(rng, D, F)
    x = rng.normal(0, 1, D).astype(np.float32)
    r1 = _shard(pkg, 4, rank, world)      # W1 gate: rows split
    r2 = _shard(pkg, 5, rank, world)      # W2 down: columns split
    w1s = w1.reshape(F, D // 32, 18)[r1[4]:r1[4] + r1[0]].reshape(-1)
    h_local = O.gemv(x, w1s, O.FMT_Q4_0, r1[0], D)[0]
    w2s = w2.reshape(D, F // 32, 18)[:, r2[5] // 32:(r2[5] + r2[1]) // 32].reshape(-1)
    part = O.gemv(h_local, np.ascontiguousarray(w2s), O.FMT_Q4_0, D, r2[1])[0].astype(np.float64)
    if rank == 0:
        total = part.copy()
        for c in ranks.peers:
            total += np.frombuffer(ranks._recv(c, D * 8), np.float64)
        full = O.gemv(O.gemv(x, w1, O.FMT_Q4_0, F, D)[0], w2, O.FMT_Q4_0, D, F)[0]
        err = float(np.abs(total - full).max() / np.abs(full).max())
        q.put((rank, got == bytes(range(128)), mx, err, r1, r2))
    else:
        ranks.sock.sendall(part.tobytes())
        q.put((rank, got == bytes(range(128)), mx, None, r1, r2))


def test_two_rank_rendezvous_and_tensor_parallel_algebra():
    pkg = load_package()
    pkg.build()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 24000 + os.getpid() % 5000
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    (_, ok0, mx0, err, a1, a2), (_, ok1, _, _, b1, b2) = res
    assert ok0 and ok1                     # both ranks hold the id made on rank 0
    assert mx0 == 11.0                     # rank 0 sees the maximum of the per-rank timings
    assert err < 1e-6                      # sharded product + sum over ranks == unsharded product
    F, D = CFG["hidden_dim"], CFG["dim"]
    assert a1[:4] == [F // 2, D, F, D] and b1[4] == F // 2 and a1[4] == 0            # gate: rows split
    assert a2[:4] == [D, F // 2, D, F] and b2[5] == F // 2 and a2[5] == 0            # down: whole blocks of K split


def test_exchange_tags_grow_and_halves_alternate():
    """The rules the fused tensor-parallel exchange relies on (include/greta_cuda.h): tags ((pos + 1) << 8) | idx are
    never zero (a cleared slot matches nothing), grow strictly along a decode session, and the exchanges of a step
    (O-projection 2l, down-projection 2l + 1, the last down-projection left to the all-reduce) alternate slot halves."""
    layers = 32
    seq = [((pos + 1) << 8) | idx for pos in range(510, 520) for idx in range(2 * layers - 1)]
    assert all(t > 0 for t in seq) and all(b > a for a, b in zip(seq, seq[1:]))
    step = list(range(2 * layers - 1))
    assert all((a & 1) != (b & 1) for a, b in zip(step, step[1:]))
    assert max(step) < 256 and ((2047 + 1) << 8 | 255) < 2 ** 32


def test_shards_tile_every_projection():
    pkg = load_package()
    pkg.build()
    for world in (1, 2, 4):
        if CFG["num_heads_kv"] % world:
            continue
        for which in range(7):
            cover = None
            for r in range(world):
                rows, cols, grows, gcols, r0, c0 = _shard(pkg, which, r, world)
                cover = np.zeros((grows, gcols // 32), np.int32) if cover is None else cover
                assert cols % 32 == 0 and c0 % 32 == 0
                cover[r0:r0 + rows, c0 // 32:(c0 + cols) // 32] += 1
            assert (cover == 1).all()


def test_peer_allreduce_protocol_model():
    """A numpy model of greta_cuda_peer_allreduce_f32 (gemv.cu, peer_allreduce_kernel): per exchange, region A of a rank's
    slot buffer holds [tp][count / tp] tagged words (row r: rank r's share of the slice this rank owns), region B holds
    [count] tagged sums; two sets alternate with the exchange index.  The model runs tp ranks through scatter, sum in rank
    order and gather for a sequence of exchanges in which one rank always races one exchange ahead of the others, and checks
    that every rank ends with the same bits, that a set is never read while a rank may still write the next-but-one
    exchange into it, and that the slot size the library reports holds both sets."""
    rng = np.random.default_rng(3)
    tp, count = 4, 4 * 96
    slice_ = count // tp
    words = 4 * count                                                     # greta_cuda_peer_allreduce_slot_bytes(count) / 8
    vals = [np.zeros((tp, words), np.float32) for _ in range(1)][0]
    tags = np.zeros((tp, words), np.int64)

    def set_off(idx):
        return (idx & 1) * 2 * count

    def phase_a(rank, x, idx, tag):
        for owner in range(tp):
            dst = set_off(idx) + rank * slice_
            vals[owner, dst:dst + slice_] = x[owner * slice_:(owner + 1) * slice_]
            tags[owner, dst:dst + slice_] = tag

    def phase_b(rank, idx, tag):
        base = set_off(idx)
        rows = np.stack([vals[rank, base + r * slice_: base + (r + 1) * slice_] for r in range(tp)])
        assert all((tags[rank, base + r * slice_: base + (r + 1) * slice_] == tag).all() for r in range(tp)), "a row was not there yet"
        v = np.zeros(slice_, np.float32)
        for r in range(tp):                                               # rank order, fp32
            v = v + rows[r]
        for j in range(tp):
            dst = base + count + rank * slice_
            vals[j, dst:dst + slice_] = v
            tags[j, dst:dst + slice_] = tag

    def phase_c(rank, idx, tag):
        base = set_off(idx) + count
        assert (tags[rank, base:base + count] == tag).all()
        return vals[rank, base:base + count].copy()

    pos = 17
    for idx in range(6):                                                   # consecutive exchanges of one decode step
        tag = ((pos + 1) << 8) | idx
        xs = [rng.normal(0, 1, count).astype(np.float32) for _ in range(tp)]
        for r in range(tp):
            phase_a(r, xs[r], idx, tag)
        for r in range(tp):
            phase_b(r, idx, tag)
        # rank 0 races ahead: it finishes this exchange and scatters the next one before the others have collected
        first = phase_c(0, idx, tag)
        ahead = rng.normal(0, 1, count).astype(np.float32)
        phase_a(0, ahead, idx + 1, ((pos + 1) << 8) | (idx + 1))           # goes into the other set
        outs = [first] + [phase_c(r, idx, tag) for r in range(1, tp)]      # the set being read is untouched
        want = np.zeros(count, np.float32)
        for r in range(tp):
            want = want + xs[r]
        assert all(np.array_equal(o.view(np.uint32), want.view(np.uint32)) for o in outs)
    assert 2 * (2 * count) <= words                                        # two sets of (region A + region B)

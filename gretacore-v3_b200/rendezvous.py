"""Multi-process glue for tensor parallelism, one process per GPU: a small TCP rendezvous on MASTER_ADDR
(hand-out of the NCCL id, barriers, gathering per-rank timings) and the set-up of the fused exchange over peer
memory (every rank's slot buffer mapped into every other rank through the C ABI's IPC calls).  No compute here."""
import os
import socket
import struct
import sys
import time

from . import ffi, model


class Ranks:
    """Tiny TCP star on MASTER_ADDR for the NCCL id hand-out and for gathering per-rank timings."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", str(self.rank)))
        self.addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        self.port = int(os.environ.get("MASTER_PORT", "29500")) + 1000
        self.peers = []
        if self.world > 1:
            if self.rank == 0:
                srv = socket.socket()
                srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
                srv.bind((self.addr, self.port))
                srv.listen(self.world)
                conns = {}
                while len(conns) < self.world - 1:
                    c, _ = srv.accept()
                    r = struct.unpack("<i", self._recv(c, 4))[0]
                    conns[r] = c
                self.peers = [conns[r] for r in sorted(conns)]
                srv.close()
            else:
                for _ in range(600):
                    try:
                        self.sock = socket.create_connection((self.addr, self.port), timeout=5)
                        break
                    except OSError:
                        time.sleep(0.1)
                else:
                    raise RuntimeError("rank 0 not reachable")
                self.sock.settimeout(None)
                self.sock.sendall(struct.pack("<i", self.rank))

    @staticmethod
    def _recv(c, n):
        buf = b""
        while len(buf) < n:
            chunk = c.recv(n - len(buf))
            if not chunk:
                raise RuntimeError("peer closed")
            buf += chunk
        return buf

    def bcast(self, data, n):
        if self.world == 1:
            return data
        if self.rank == 0:
            for c in self.peers:
                c.sendall(data)
            return data
        return self._recv(self.sock, n)

    def gather_max(self, value):
        if self.world == 1:
            return value
        if self.rank == 0:
            vals = [value] + [struct.unpack("<d", self._recv(c, 8))[0] for c in self.peers]
            return max(vals)
        self.sock.sendall(struct.pack("<d", value))
        return value

    def barrier(self):
        self.gather_max(0.0)
        self.bcast(b"go!!", 4)

    def allgather(self, data):
        """Every rank contributes len(data) bytes; returns the list of all ranks' contributions."""
        n = len(data)
        if self.world == 1:
            return [data]
        if self.rank == 0:
            parts = [data] + [self._recv(c, n) for c in self.peers]
            self.bcast(b"".join(parts), n * self.world)
            return parts
        self.sock.sendall(data)
        blob = self._recv(self.sock, n * self.world)
        return [blob[i * n:(i + 1) * n] for i in range(self.world)]


def install_peer_exchange(mdl, ranks, dim, batch=1):
    """Sets up the fused tensor-parallel exchange: every rank allocates its slot buffer, the processes swap the
    64-byte IPC handles over the rendezvous sockets, map each other's buffers and hand the table to the model.
    Returns the objects that must stay alive (local buffer, descriptor, mapped pointers), or None - on every rank
    alike - when any rank could not export or map a buffer (the model then keeps the all-reduce)."""
    import ctypes as C
    g = ffi
    lib = g.cuda()
    local, handle, ok = None, C.create_string_buffer(64), True
    try:
        nbytes = lib.greta_cuda_peer_slot_bytes(ranks.world, dim)
        if batch > 1:                                                 # room for the all-reduce of [batch x dim] through peer memory
            nbytes = max(nbytes, lib.greta_cuda_peer_allreduce_slot_bytes(batch * dim))
        local = g.DeviceBuffer(nbytes, zero=True)
        g.check(lib.greta_cuda_ipc_export(local.ptr, handle), "ipc_export")
    except Exception as e:                                            # noqa: BLE001 - reported, then agreed on by all ranks
        print(f"rank {ranks.rank}: peer exchange unavailable: {e}", file=sys.stderr)
        ok = False
    got = ranks.allgather(bytes(handle.raw) + (b"\1" if ok else b"\0"))
    if not all(h[64:] == b"\1" for h in got):
        return None
    ex = model.PeerExchange()
    ex.tp, ex.rank, ex.slot_bytes = ranks.world, ranks.rank, nbytes
    mapped = []
    try:
        for r, h in enumerate(got):
            if r == ranks.rank:
                ex.slots[r] = local.ptr
            else:
                ptr = C.c_void_p()
                g.check(lib.greta_cuda_ipc_open(C.create_string_buffer(h[:64], 64), C.byref(ptr)), "ipc_open")
                ex.slots[r] = ptr.value
                mapped.append(ptr.value)
    except Exception as e:                                            # noqa: BLE001
        print(f"rank {ranks.rank}: peer exchange unavailable: {e}", file=sys.stderr)
        ok = False
    if not all(f == b"\1" for f in ranks.allgather(b"\1" if ok else b"\0")):   # also: every buffer is cleared and mapped from here on
        for ptr in mapped:
            lib.greta_cuda_ipc_close(ptr)
        return None
    mdl.set_peer_exchange(ex)
    return local, ex, mapped

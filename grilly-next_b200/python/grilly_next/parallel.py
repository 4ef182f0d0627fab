"""Long-context decode with the KV sequence sharded over GPUs (one process per GPU).

Rank g of G holds the contiguous token range shard_range(T, G, g) of every sequence in its own
paged cache.  A step is: every rank runs split-KV decode over its shard and leaves ONE
un-normalised partial [O (rows*D) | m (rows) | l (rows)] (grl_gqa_decode with partial_out), the
partials cross NVLink (16,640 bytes per rank at B=1, Hq=32, D=128) and every rank merges them with
the log-sum-exp merge.  This is the only exchange on the attention path; batch / head partitioning
of the other workloads needs none.  Four interchangeable forms of the exchange, all behind the C ABI:

  "nccl"    grl_group_allgather_merge: NCCL all-gather, then the merge kernel
  "merge"   grl_exchange_merge, flag form: peer stores + fence + flag, bounded wait, merge -- one kernel
  "ll"      grl_exchange_merge, {value, step} pair form: no fence and no flag
  "decode"  grl_gqa_decode with `exchange`: decode, exchange and merge in ONE launch

The reference has no multi-GPU code at all; the decomposition follows the split-KV scheme of its
decode shader's CPU twin (tests/test_inference_ops.py:64-95) applied across devices.

Nothing here needs a framework: ranks meet over a HostChannel (any object with rank, world,
all_gather_bytes and barrier -- TcpChannel below is one over plain sockets), device memory comes from
the C ABI.  The mode logic is backend-agnostic (`ops` supplies the kernels), so the same class runs
on CPU in the tests with numpy stand-ins for the kernels.
"""
from __future__ import annotations

import ctypes as C
import socket
import struct
import time


def shard_range(total_tokens: int, world: int, rank: int):
    """Contiguous [start, end) of rank's tokens; the first (total % world) ranks get one more."""
    base, rem = divmod(int(total_tokens), int(world))
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def owner_of_new_token(world: int) -> int:
    """New tokens of a growing sequence are appended on the last rank (its range is the tail)."""
    return world - 1


def partial_floats(rows: int, head_dim: int) -> int:
    return rows * (head_dim + 2)


class SingleChannel:
    """The channel of a lone process."""
    rank, world = 0, 1

    def all_gather_bytes(self, payload: bytes):
        return [payload]

    def barrier(self):
        pass


class TcpChannel:
    """Host-side meeting point of the ranks over plain TCP: rank 0 listens, the others connect.

    Only small control messages travel here (the NCCL id, CUDA IPC handles, barriers, timings);
    data goes over NVLink.  all_gather_bytes returns every rank's payload, in rank order.
    """

    def __init__(self, rank: int, world: int, addr: str = "127.0.0.1", port: int = 29611, timeout_s: float = 120.0):
        self.rank, self.world = int(rank), int(world)
        self._peers = []
        self._sock = None
        if self.world == 1:
            return
        if self.rank == 0:
            srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            srv.bind((addr, port))
            srv.listen(self.world)
            srv.settimeout(timeout_s)
            conns = {}
            while len(conns) < self.world - 1:
                c, _ = srv.accept()
                c.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
                c.settimeout(timeout_s)
                (r,) = struct.unpack("<i", self._recv_exact(c, 4))
                conns[r] = c
            srv.close()
            self._peers = [conns[r] for r in range(1, self.world)]
        else:
            deadline = time.time() + timeout_s
            while True:
                try:
                    s = socket.create_connection((addr, port), timeout=timeout_s)
                    break
                except OSError:
                    if time.time() > deadline:
                        raise
                    time.sleep(0.05)
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            s.settimeout(timeout_s)
            s.sendall(struct.pack("<i", self.rank))
            self._sock = s

    @staticmethod
    def _recv_exact(sock, n):
        buf = bytearray()
        while len(buf) < n:
            chunk = sock.recv(n - len(buf))
            if not chunk:
                raise ConnectionError("peer closed the channel")
            buf += chunk
        return bytes(buf)

    @classmethod
    def _send_msg(cls, sock, payload: bytes):
        sock.sendall(struct.pack("<q", len(payload)) + payload)

    @classmethod
    def _recv_msg(cls, sock) -> bytes:
        (n,) = struct.unpack("<q", cls._recv_exact(sock, 8))
        return cls._recv_exact(sock, n)

    def all_gather_bytes(self, payload: bytes):
        payload = bytes(payload)
        if self.world == 1:
            return [payload]
        if self.rank == 0:
            parts = [payload] + [self._recv_msg(c) for c in self._peers]
            blob = b"".join(struct.pack("<q", len(p)) + p for p in parts)
            for c in self._peers:
                self._send_msg(c, blob)
            return parts
        self._send_msg(self._sock, payload)
        blob = self._recv_msg(self._sock)
        parts, off = [], 0
        for _ in range(self.world):
            (n,) = struct.unpack_from("<q", blob, off)
            parts.append(blob[off + 8: off + 8 + n])
            off += 8 + n
        return parts

    def barrier(self):
        self.all_gather_bytes(b"")

    def close(self):
        for c in self._peers:
            c.close()
        if self._sock:
            self._sock.close()
        self._peers, self._sock = [], None


def max_over_ranks(channel, value: float) -> float:
    return max(struct.unpack("<d", b)[0] for b in channel.all_gather_bytes(struct.pack("<d", float(value))))


class ShardedDecoder:
    """Chooses the form of a step.  `ops` supplies: full(q) (one GPU holds everything), partial(q),
    allgather_merge(part) (collective form), and optionally decode_exchange(q) / exchange_merge()
    with the flags p2p_ready / one_launch (peer-memory forms)."""

    def __init__(self, channel, ops):
        self.channel, self.ops = channel, ops
        self.world, self.rank = channel.world, channel.rank

    def step(self, q):
        if self.world == 1 and hasattr(self.ops, "full"):
            return self.ops.full(q)          # one GPU holds everything: normalised output directly
        if self.world > 1 and getattr(self.ops, "p2p_ready", False) and getattr(self.ops, "one_launch", False):
            return self.ops.decode_exchange(q)   # decode, NVLink exchange and merge in ONE kernel launch
        part = self.ops.partial(q)
        if self.world > 1 and getattr(self.ops, "p2p_ready", False):
            return self.ops.exchange_merge()     # partials cross NVLink inside the merge kernel, no collective call
        return self.ops.allgather_merge(part)    # NCCL all-gather + merge (a single rank: merge of one part)


class CudaShardOps:
    """The kernels of a step through the C ABI, on the stream of `dev` (a cabi.Device).

    `layout` is the grl_kv_layout of this rank's shard; q is a device pointer (ctypes.c_void_p) to
    (B,1,Hq,D) float32; every method returns the device pointer of the (B,1,Hq,D) float32 result.
    """

    def __init__(self, cabi, dev, layout, num_q_heads, max_seq_len, n_splits=0):
        self.cabi, self.dev = cabi, dev
        self.Hq, self.D, self.B = num_q_heads, layout.head_dim, layout.batch
        self.rows = self.B * self.Hq
        p = cabi.DecodeParams()
        p.kv, p.num_q_heads, p.max_seq_len, p.n_splits = layout, num_q_heads, max(1, max_seq_len), n_splits
        ns = C.c_int()
        cabi.check(dev.L.grl_decode_pick_splits(dev.h, C.byref(p), C.byref(ns)))
        wb = C.c_size_t()
        cabi.check(dev.L.grl_decode_workspace_bytes(C.byref(p), ns.value, C.byref(wb)))
        self.ws = dev.malloc(max(wb.value, 256))
        p.n_splits, p.workspace, p.workspace_bytes = ns.value, self.ws, wb.value
        self.p = p
        n = partial_floats(self.rows, self.D)
        self.part = dev.malloc(n * 4)
        self.out = dev.malloc(self.rows * self.D * 4)
        self.group, self.gathered = None, None
        self.p2p_ready, self.one_launch = False, False

    # ---- collective form
    def setup_nccl(self, channel):
        """Collective: rank 0 makes the NCCL id, the channel carries it, every rank joins."""
        cabi, dev = self.cabi, self.dev
        raw = b""
        if channel.rank == 0:
            buf = (C.c_char * 128)()
            cabi.check(dev.L.grl_group_unique_id(buf))
            raw = bytes(buf)
        raw = channel.all_gather_bytes(raw)[0]
        g = C.c_void_p()
        cabi.check(dev.L.grl_group_init_rank(dev.h, C.create_string_buffer(raw, 128), channel.rank, channel.world, C.byref(g)))
        self.group = g
        self.gathered = dev.malloc(channel.world * partial_floats(self.rows, self.D) * 4)

    def allgather_merge(self, part=None):
        if self.group is None:      # a lone rank without a group: the merge of one part normalises it
            self.cabi.check(self.dev.L.grl_lse_merge(self.dev.h, self.part, 1, partial_floats(self.rows, self.D),
                                                     self.rows, self.D, 1, self.out))
            return self.out
        self.cabi.check(self.dev.L.grl_group_allgather_merge(self.group, self.part, self.rows, self.D, self.gathered,
                                                             self.out, 0))
        return self.out

    # ---- peer-memory forms
    def setup_p2p(self, channel, one_launch=True, low_latency=True, wait_cycles=0):
        """Map every peer's inbox into this process (CUDA IPC) for the fused exchange + merge kernels.
        Collective: every rank calls it once.  p2p_ready stays False if a handle cannot be opened, e.g.
        without peer access between the GPUs."""
        cabi, dev, L = self.cabi, self.dev, self.dev.L
        world, rank = channel.world, channel.rank
        n = partial_floats(self.rows, self.D)
        inbox_bytes = 2 * world * n * (8 if low_latency else 4)   # low latency: {value, step} pairs
        self._inbox = dev.malloc(inbox_bytes)
        slots = self.B * self.p.kv.num_kv_heads
        flag_bytes = 2 * world * slots * 4 + 64
        self._flags = dev.malloc(flag_bytes)
        self._seq = dev.malloc(64)
        for p_, nb in ((self._inbox, inbox_bytes), (self._flags, flag_bytes), (self._seq, 64)):
            cabi.check(L.grl_memset(dev.h, p_, 0, nb))
        dev.sync()
        hi, hf = (C.c_char * 64)(), (C.c_char * 64)()
        cabi.check(L.grl_ipc_export(dev.h, self._inbox, hi))
        cabi.check(L.grl_ipc_export(dev.h, self._flags, hf))
        handles = channel.all_gather_bytes(bytes(hi) + bytes(hf))
        self._peer_inbox = (C.c_void_p * world)()
        self._peer_flags = (C.c_void_p * world)()
        ok = True
        for r in range(world):
            if r == rank:
                continue
            for raw, table in ((handles[r][:64], self._peer_inbox), (handles[r][64:], self._peer_flags)):
                ptr = C.c_void_p()
                if L.grl_ipc_import(dev.h, C.create_string_buffer(raw, 64), C.byref(ptr)) != 0:
                    ok = False
                table[r] = ptr.value
        all_ok = channel.all_gather_bytes(b"\x01" if ok else b"\x00")   # also the barrier: nobody stores into an
        self.p2p_ready = all(b == b"\x01" for b in all_ok)               # inbox before everybody has zeroed it
        e = cabi.ExchangeParams()
        e.local_partial, e.inbox, e.flags = self.part, self._inbox, self._flags
        e.peer_inbox = C.cast(self._peer_inbox, C.POINTER(C.c_void_p))
        e.peer_flags = C.cast(self._peer_flags, C.POINTER(C.c_void_p))
        e.seq, e.out = self._seq, self.out
        e.rank, e.world, e.rows, e.head_dim, e.flag_slots = rank, world, self.rows, self.D, slots
        e.low_latency = int(low_latency)
        e.wait_cycles = int(wait_cycles)
        self._exchange = e
        # the decode kernel itself can do the exchange for the tensor-core geometry with few enough heads
        self.one_launch = bool(one_launch and low_latency and self.p.kv.cache_dtype == cabi.BF16 and self.D == 128
                               and self.p.kv.page_tokens == 64 and slots <= 128)
        return self.p2p_ready

    def reset_exchange(self):
        """After a GRL_ERR_TIMEOUT: every rank calls this, then the ranks meet at a barrier."""
        self.cabi.check(self.dev.L.grl_exchange_reset(self.dev.h, C.byref(self._exchange)))

    def decode_exchange(self, q):
        self.p.q, self.p.out, self.p.partial_out = q, self.out, None
        self.p.exchange = C.pointer(self._exchange)
        try:
            self.cabi.check(self.dev.L.grl_gqa_decode(self.dev.h, C.byref(self.p)))
        finally:
            self.p.exchange = None
        return self.out

    def exchange_merge(self):
        self.cabi.check(self.dev.L.grl_exchange_merge(self.dev.h, C.byref(self._exchange)))
        return self.out

    def set_layout(self, layout):
        self.p.kv = layout

    def partial(self, q):
        self.p.q, self.p.out, self.p.partial_out = q, None, self.part
        self.cabi.check(self.dev.L.grl_gqa_decode(self.dev.h, C.byref(self.p)))
        return self.part

    def full(self, q):
        self.p.q, self.p.out, self.p.partial_out = q, self.out, None
        self.cabi.check(self.dev.L.grl_gqa_decode(self.dev.h, C.byref(self.p)))
        return self.out

    def close(self):
        """Collective when a group exists (the communicator is destroyed)."""
        if self.group is not None:
            self.dev.sync()
            self.dev.L.grl_group_destroy(self.group)
            self.group = None

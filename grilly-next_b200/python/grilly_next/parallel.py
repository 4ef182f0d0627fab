"""Long-context decode with the KV sequence sharded over GPUs (one process per GPU).

Rank g of G holds the contiguous token range shard_range(T, G, g) of every sequence in its own
paged cache.  A step is: every rank runs split-KV decode over its shard and leaves ONE
un-normalised partial [O (rows*D) | m (rows) | l (rows)] (grl_gqa_decode with partial_out), the
partials are all-gathered (NCCL over NVLink on GPUs; 16,640 bytes per rank at B=1, Hq=32, D=128),
and every rank merges them with the log-sum-exp merge (grl_lse_merge).  This is the only collective
on the attention path; batch / head partitioning of the other workloads needs none.

The reference has no multi-GPU code at all; the decomposition follows the split-KV scheme of its
decode shader's CPU twin (tests/test_inference_ops.py:64-95) applied across devices.

The collective and the sharding arithmetic are backend-agnostic (`ops` supplies the two kernels), so
the same class runs over gloo on CPU in the tests, with numpy stand-ins for the kernels.
"""
from __future__ import annotations

import ctypes as C


def shard_range(total_tokens: int, world: int, rank: int):
    """Contiguous [start, end) of rank's tokens; the first (total % world) ranks get one more."""
    base, rem = divmod(int(total_tokens), int(world))
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def owner_of_new_token(world: int) -> int:
    """New tokens of a growing sequence are appended on the last rank (its range is the tail)."""
    return world - 1


def torch_stream_handle(torch):
    """torch's current CUDA stream as a handle for grl_device_use_stream.  The legacy default stream's
    handle is NULL, which the library reads as "back to your own stream": name it as cudaStreamLegacy."""
    h = torch.cuda.current_stream().cuda_stream
    return C.c_void_p(h if h else 1)


def partial_floats(rows: int, head_dim: int) -> int:
    return rows * (head_dim + 2)


class ShardedDecoder:
    """ops.partial(q) -> 1-D float tensor of partial_floats(); ops.merge(gathered 2-D, n_parts) -> output.

    `dist` is torch.distributed (initialised by the caller: nccl on GPUs, gloo in the CPU tests);
    `empty(n_parts, n)` allocates the gather buffer on the backend's device.
    """

    def __init__(self, dist, ops, empty):
        self.dist, self.ops, self.empty = dist, ops, empty
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self._gather = None

    def step(self, q):
        if self.world == 1 and hasattr(self.ops, "full"):
            return self.ops.full(q)          # one GPU holds everything: normalised output directly
        if self.world > 1 and getattr(self.ops, "p2p_ready", False) and getattr(self.ops, "one_launch", False):
            return self.ops.decode_exchange(q)   # decode, NVLink exchange and merge in ONE kernel launch
        part = self.ops.partial(q)
        if self.world == 1:
            return self.ops.merge(part.reshape(1, -1), 1)
        if getattr(self.ops, "p2p_ready", False):
            return self.ops.exchange_merge()     # partials cross NVLink inside the merge kernel, no collective call
        if self._gather is None or self._gather.shape[1] != part.numel():
            self._gather = self.empty(self.world, part.numel())
        self.dist.all_gather_into_tensor(self._gather.reshape(-1), part)
        return self.ops.merge(self._gather, self.world)


class CudaShardOps:
    """The two kernels of a step through the C ABI, on torch's current CUDA stream.

    `dev` is a cabi.Device whose stream was set with grl_device_use_stream(torch_stream_handle(torch)), so that
    the kernels are ordered with torch's NCCL calls; `layout`
    the grl_kv_layout of this rank's shard; q / outputs are torch CUDA float32 tensors.
    """

    def __init__(self, cabi, dev, layout, num_q_heads, max_seq_len, torch, n_splits=0):
        self.cabi, self.dev, self.torch = cabi, dev, torch
        self.Hq, self.D, self.B = num_q_heads, layout.head_dim, layout.batch
        self.rows = self.B * self.Hq
        p = cabi.DecodeParams()
        p.kv, p.num_q_heads, p.max_seq_len, p.n_splits = layout, num_q_heads, max_seq_len, n_splits
        ns = C.c_int()
        cabi.check(dev.L.grl_decode_pick_splits(dev.h, C.byref(p), C.byref(ns)))
        wb = C.c_size_t()
        cabi.check(dev.L.grl_decode_workspace_bytes(C.byref(p), ns.value, C.byref(wb)))
        self.ws = torch.empty(max(wb.value, 16) // 4, dtype=torch.float32, device="cuda")
        p.n_splits, p.workspace, p.workspace_bytes = ns.value, self.ws.data_ptr(), wb.value
        self.p = p
        self.part = torch.empty(partial_floats(self.rows, self.D), dtype=torch.float32, device="cuda")
        self.out = torch.empty((self.B, 1, self.Hq, self.D), dtype=torch.float32, device="cuda")

    def setup_p2p(self, dist, one_launch=True, low_latency=True):
        """Map every peer's inbox into this process (CUDA IPC) for the fused exchange + merge kernel.
        Collective: every rank calls it once.  Falls back silently (p2p_ready stays False) if the
        handles cannot be opened, e.g. without peer access between the GPUs."""
        cabi, dev, L = self.cabi, self.dev, self.dev.L
        world, rank = dist.get_world_size(), dist.get_rank()
        n = partial_floats(self.rows, self.D)
        inbox_bytes = 2 * world * n * (8 if low_latency else 4)   # low latency: {value, step} pairs
        self._inbox = dev.malloc(inbox_bytes)
        slots = self.B * self.p.kv.num_kv_heads          # one flag per (sequence, kv head): heads cross as they finish
        self._flags = dev.malloc(2 * world * slots * 4 + 64)
        self._seq = dev.malloc(64)
        for p_, nb in ((self._inbox, inbox_bytes), (self._flags, 2 * world * slots * 4 + 64), (self._seq, 64)):
            cabi.check(L.grl_memset(dev.h, p_, 0, nb))
        dev.sync()
        hi, hf = (C.c_char * 64)(), (C.c_char * 64)()
        cabi.check(L.grl_ipc_export(dev.h, self._inbox, hi))
        cabi.check(L.grl_ipc_export(dev.h, self._flags, hf))
        mine = (bytes(hi), bytes(hf))
        handles = [None] * world
        dist.all_gather_object(handles, mine)
        self._peer_inbox = (C.c_void_p * world)()
        self._peer_flags = (C.c_void_p * world)()
        ok = True
        for r in range(world):
            if r == rank:
                continue
            for raw, table in ((handles[r][0], self._peer_inbox), (handles[r][1], self._peer_flags)):
                ptr = C.c_void_p()
                if L.grl_ipc_import(dev.h, C.create_string_buffer(raw, 64), C.byref(ptr)) != 0:
                    ok = False
                table[r] = ptr.value
        all_ok = [None] * world
        dist.all_gather_object(all_ok, ok)
        dist.barrier()            # nobody stores into an inbox before everybody has zeroed and exported it
        self.p2p_ready = all(all_ok)
        e = cabi.ExchangeParams()
        e.local_partial, e.inbox, e.flags = self.part.data_ptr(), self._inbox, self._flags
        e.peer_inbox = C.cast(self._peer_inbox, C.POINTER(C.c_void_p))
        e.peer_flags = C.cast(self._peer_flags, C.POINTER(C.c_void_p))
        e.seq, e.out = self._seq, self.out.data_ptr()
        e.rank, e.world, e.rows, e.head_dim, e.flag_slots = rank, world, self.rows, self.D, slots
        e.low_latency = int(low_latency)
        self._exchange = e
        # the decode kernel itself can do the exchange for the tensor-core geometry with few enough heads
        self.one_launch = bool(one_launch and low_latency and self.p.kv.cache_dtype == cabi.BF16 and self.D == 128
                               and self.p.kv.page_tokens == 64 and slots <= 128)
        return self.p2p_ready

    def decode_exchange(self, q):
        self.p.q, self.p.out, self.p.partial_out = q.data_ptr(), self.out.data_ptr(), None
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
        self.p.q, self.p.out, self.p.partial_out = q.data_ptr(), None, self.part.data_ptr()
        self.cabi.check(self.dev.L.grl_gqa_decode(self.dev.h, C.byref(self.p)))
        return self.part

    def full(self, q):
        self.p.q, self.p.out, self.p.partial_out = q.data_ptr(), self.out.data_ptr(), None
        self.cabi.check(self.dev.L.grl_gqa_decode(self.dev.h, C.byref(self.p)))
        return self.out

    def merge(self, gathered, n_parts):
        self.cabi.check(self.dev.L.grl_lse_merge(self.dev.h, gathered.data_ptr(), n_parts,
                                                 partial_floats(self.rows, self.D), self.rows, self.D, 1,
                                                 self.out.data_ptr()))
        return self.out

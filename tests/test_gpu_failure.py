"""Failure paths of the device-side waits, made to happen on the host side only.

The reference reports a stuck submission through a 2 s fence timeout that becomes a std::runtime_error
(cpp/src/command_batch.cpp:16,145-148).  Here every wait inside a kernel has a cycle budget; when it runs
out the kernel RETURNS and leaves GRL_ERR_TIMEOUT in the device's status word, which the next grl_sync
reports.  These tests make a wait run out without faulting, trapping or hanging anything: the cross-GPU
merge is run with world = 2 on ONE device, its "peer" being a second local buffer that nobody ever writes,
with a budget of about a millisecond.  Afterwards the same device must serve an ordinary decode.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SHORT_WAIT = 2_000_000      # cycles: about 1 ms


def _exchange_params(dev, cabi, rows, D, low_latency, part=None, out=None):
    """world = 2, this rank 0; rank 1's inbox and flags are local buffers that stay zero."""
    n = rows * (D + 2)
    esz = 8 if low_latency else 4
    bufs = {
        "inbox": dev.malloc(2 * 2 * n * esz), "flags": dev.malloc(2 * 2 * 8 * 4 + 64), "seq": dev.malloc(64),
        "peer_inbox": dev.malloc(2 * 2 * n * esz), "peer_flags": dev.malloc(2 * 2 * 8 * 4 + 64),
    }
    for k, nb in (("inbox", 2 * 2 * n * esz), ("flags", 2 * 2 * 8 * 4 + 64), ("seq", 64), ("peer_inbox", 2 * 2 * n * esz),
                  ("peer_flags", 2 * 2 * 8 * 4 + 64)):
        cabi.check(dev.L.grl_memset(dev.h, bufs[k], 0, nb))
    e = cabi.ExchangeParams()
    peers_i, peers_f = (C.c_void_p * 2)(), (C.c_void_p * 2)()
    peers_i[1], peers_f[1] = bufs["peer_inbox"].value, bufs["peer_flags"].value
    e.local_partial, e.inbox, e.flags, e.seq, e.out = part, bufs["inbox"], bufs["flags"], bufs["seq"], out
    e.peer_inbox = C.cast(peers_i, C.POINTER(C.c_void_p))
    e.peer_flags = C.cast(peers_f, C.POINTER(C.c_void_p))
    e.rank, e.world, e.rows, e.head_dim, e.flag_slots, e.low_latency = 0, 2, rows, D, 8, int(low_latency)
    e.wait_cycles = SHORT_WAIT
    e._keep = (peers_i, peers_f, bufs)
    return e


def _ordinary_decode_passes(dev, cabi):
    from gpu_helpers import PagedCache
    from oracle import attention_oracle as orc
    rng = np.random.default_rng(5)
    B, Hq, Hkv, D, T = 1, 8, 2, 128, 700
    k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
    pc = PagedCache(dev, B, Hkv, D, 768, dtype=cabi.BF16)
    pc.append(k, v)
    got = pc.decode(q, n_splits=3)
    want = orc.gqa_decode_attention(q, orc.round_bf16(k), orc.round_bf16(v), Hq, Hkv, D)
    assert np.abs(got - want).max() <= 5e-3


@pytest.mark.parametrize("low_latency", [False, True])
def test_exchange_wait_runs_out_and_the_device_stays_usable(low_latency):
    from grilly_next import cabi
    dev = cabi.Device(0)
    try:
        rows, D = 8, 128
        rng = np.random.default_rng(1)
        part = dev.upload(rng.standard_normal(rows * (D + 2)).astype(np.float32))
        out = dev.malloc(rows * D * 4)
        e = _exchange_params(dev, cabi, rows, D, low_latency, part, out)
        cabi.check(dev.L.grl_exchange_merge(dev.h, C.byref(e)))
        rc = dev.L.grl_sync(dev.h, 0)
        assert rc == cabi.ERR_TIMEOUT, dev.L.grl_last_error()
        msg = dev.L.grl_last_error().decode()
        assert "peer 1" in msg, msg                      # the rank that never posted
        cabi.check(dev.L.grl_exchange_reset(dev.h, C.byref(e)))
        dev.sync()                                       # the status word was cleared with the report
        assert dev.download(e.seq, (1,), np.uint32)[0] == 0
        _ordinary_decode_passes(dev, cabi)
    finally:
        dev.close()


def test_fused_decode_exchange_times_out_in_a_replayed_graph():
    """Decode + exchange in one launch, captured in a graph: the replay's timeout must reach grl_sync too."""
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    dev = cabi.Device(0)
    try:
        rng = np.random.default_rng(2)
        B, Hq, Hkv, D, T = 1, 32, 8, 128, 1500
        pc = PagedCache(dev, B, Hkv, D, 1536, dtype=cabi.BF16)
        pc.append(rng.standard_normal((B, T, Hkv, D), dtype=np.float32), rng.standard_normal((B, T, Hkv, D), dtype=np.float32))
        q = dev.upload(rng.standard_normal((B, 1, Hq, D), dtype=np.float32))
        out = dev.malloc(B * Hq * D * 4)
        cabi.check(dev.L.grl_memset(dev.h, out, 0, B * Hq * D * 4))
        e = _exchange_params(dev, cabi, B * Hq, D, True)
        p = cabi.DecodeParams()
        p.kv, p.q, p.out, p.num_q_heads, p.n_splits, p.max_seq_len = pc.layout(), q, out, Hq, 4, T
        wb = C.c_size_t()
        cabi.check(dev.L.grl_decode_workspace_bytes(C.byref(p), 4, C.byref(wb)))
        p.workspace, p.workspace_bytes = dev.malloc(wb.value), wb.value
        p.exchange = C.pointer(e)
        dev.sync()
        g = C.c_void_p()
        cabi.check(dev.L.grl_graph_begin(dev.h))
        cabi.check(dev.L.grl_gqa_decode(dev.h, C.byref(p)))
        cabi.check(dev.L.grl_graph_end(dev.h, C.byref(g)))
        dev.sync()                                       # capture launched nothing: no failure yet
        cabi.check(dev.L.grl_graph_launch(dev.h, g))
        rc = dev.L.grl_sync(dev.h, 0)
        assert rc == cabi.ERR_TIMEOUT, dev.L.grl_last_error()
        assert "peer 1" in dev.L.grl_last_error().decode()
        assert not dev.download(out, (B * Hq * D,), np.float32).any()    # no row is written after a timeout
        assert dev.download(e.seq, (1,), np.uint32)[0] == 0              # the step was not counted
        dev.L.grl_graph_destroy(g)
        cabi.check(dev.L.grl_exchange_reset(dev.h, C.byref(e)))
        dev.sync()
        _ordinary_decode_passes(dev, cabi)
    finally:
        dev.close()


def test_wait_limits_setter_and_defaults():
    from grilly_next import cabi
    dev = cabi.Device(0)
    try:
        cabi.check(dev.L.grl_device_set_wait_limits(dev.h, 5_000_000, 3_000_000))
        _ordinary_decode_passes(dev, cabi)               # generous enough for real work
        cabi.check(dev.L.grl_device_set_wait_limits(dev.h, 0, 0))
        _ordinary_decode_passes(dev, cabi)
    finally:
        dev.close()


def test_append_to_a_full_sequence_is_refused_on_the_device():
    """A C-ABI caller that appends past the block table gets an error code and an untouched cache."""
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    dev = cabi.Device(0)
    try:
        rng = np.random.default_rng(3)
        B, Hkv, D = 2, 2, 64
        pc = PagedCache(dev, B, Hkv, D, 32, page_tokens=16, dtype=cabi.F32)     # two pages per sequence
        k = rng.standard_normal((B, 32, Hkv, D), dtype=np.float32)
        pc.append(k, k)
        before = [pc.gather(b) for b in range(B)]
        more = rng.standard_normal((B, 1, Hkv, D), dtype=np.float32)
        kd = dev.upload(more)
        p = cabi.AppendParams()
        p.kv, p.k_new, p.v_new, p.n_new, p.update_lens = pc.layout(), kd, kd, 1, 1
        cabi.check(dev.L.grl_kv_append(dev.h, C.byref(p)))
        rc = dev.L.grl_sync(dev.h, 0)
        assert rc == -6, (rc, dev.L.grl_last_error())    # GRL_ERR_KERNEL: the kernel refused
        assert "no room" in dev.L.grl_last_error().decode()
        assert (dev.download(pc.seq_lens, (B,), np.int32) == 32).all()
        for b in range(B):
            kb, vb = pc.gather(b)
            assert np.array_equal(kb, before[b][0]) and np.array_equal(vb, before[b][1])
    finally:
        dev.close()


def test_tensor_maps_are_encoded_once_per_buffer():
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    dev = cabi.Device(0)
    try:
        rng = np.random.default_rng(4)
        B, Hq, Hkv, D, T = 2, 8, 2, 128, 300
        pc = PagedCache(dev, B, Hkv, D, 320, dtype=cabi.BF16)
        pc.append(rng.standard_normal((B, T, Hkv, D), dtype=np.float32), rng.standard_normal((B, T, Hkv, D), dtype=np.float32))
        qd = dev.upload(rng.standard_normal((B, 1, Hq, D), dtype=np.float32))
        od = dev.malloc(B * Hq * D * 4)
        p = cabi.DecodeParams()
        p.kv, p.q, p.out, p.num_q_heads, p.n_splits, p.max_seq_len = pc.layout(), qd, od, Hq, 1, T
        h, m, c = C.c_int64(), C.c_int64(), C.c_int64()
        cabi.check(dev.L.grl_tensor_map_cache_stats(dev.h, C.byref(h), C.byref(m), C.byref(c)))
        h0, m0 = h.value, m.value
        for _ in range(5):
            cabi.check(dev.L.grl_gqa_decode(dev.h, C.byref(p)))
        dev.sync()
        cabi.check(dev.L.grl_tensor_map_cache_stats(dev.h, C.byref(h), C.byref(m), C.byref(c)))
        assert m.value - m0 == 2 and h.value - h0 == 8      # K and V pools encoded once, found four times each
        dev.free(pc.k_pages)                                 # freeing a buffer forgets its maps
        cabi.check(dev.L.grl_tensor_map_cache_stats(dev.h, C.byref(h), C.byref(m), C.byref(c)))
        assert c.value == 1
    finally:
        dev.close()


def test_rope_table_grows_with_the_sequence_and_is_refused_inside_a_capture():
    from grilly_next import cabi
    from gpu_helpers import flash_cabi
    from oracle import attention_oracle as orc
    dev = cabi.Device(0)
    try:
        rng = np.random.default_rng(6)
        for S in (200, 700, 300):            # second call outgrows the first table, third fits the second
            Q, K, V = (rng.standard_normal((1, 2, S, 64), dtype=np.float32) for _ in range(3))
            pos = np.arange(S)
            want = orc.attention_4d(orc.rope_interleaved(Q, pos), orc.rope_interleaved(K, pos), V,
                                    mask=orc.causal_length_mask(1, 2, S, None, True))
            got = flash_cabi(dev, Q, K, V, causal=True, rope_mode=cabi.ROPE_INTERLEAVED, kernel=cabi.KERNEL_SIMT_F32)
            assert np.abs(got - want).max() <= 1e-4
        # a table that does not exist yet cannot be built while the stream is capturing
        q = dev.malloc(4096 * 64 * 4)
        p = cabi.FlashParams()
        p.q = p.k = p.v = p.o = q
        p.in_dtype, p.out_dtype, p.batch, p.heads, p.seq_len, p.head_dim = cabi.F32, cabi.F32, 1, 1, 4096, 64
        p.rope_mode, p.rope_theta, p.rope_scaling, p.kernel = cabi.ROPE_HALF, 500000.0, 1.0, cabi.KERNEL_SIMT_F32
        cabi.check(dev.L.grl_graph_begin(dev.h))
        rc = dev.L.grl_flash_fwd(dev.h, C.byref(p))
        msg = dev.L.grl_last_error().decode()
        g = C.c_void_p()
        cabi.check(dev.L.grl_graph_end(dev.h, C.byref(g)))
        dev.L.grl_graph_destroy(g)
        assert rc == -1 and "grl_rope_table_prepare" in msg
        cabi.check(dev.L.grl_rope_table_prepare(dev.h, 4096, 64, 500000.0, 1.0))
        dev.sync()
    finally:
        dev.close()

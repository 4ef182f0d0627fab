"""grl_gqa_decode_static: the decode step for hosts that may not allocate device memory.

A serving process that gave all device memory to its own arena, or a plugin that is handed only its
input and output tensors, cannot pass the split-KV workspace that grl_gqa_decode wants.  The static
entry point keeps the partials in an array inside the library instead.  Here it is called through
the C ABI next to the ordinary entry point, twice in a row on different data (the array keeps the
first call's contents), and asked for more scratch than it has.

Runs last on purpose (file name): a failure here cannot hide another test's result.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _decode_both(dev, pc, q, n_splits):
    from grilly_next import cabi
    B, _, Hq, D = q.shape
    qd = dev.upload(q)
    out_ws, out_st = dev.malloc(q.nbytes), dev.malloc(q.nbytes)
    p = cabi.DecodeParams()
    p.kv = pc.layout()
    p.q, p.num_q_heads, p.n_splits, p.max_seq_len = qd, Hq, n_splits, int(pc.lens.max())
    wb = C.c_size_t()
    cabi.check(dev.L.grl_decode_workspace_bytes(C.byref(p), n_splits, C.byref(wb)))
    ws = dev.malloc(wb.value)
    p.out, p.workspace, p.workspace_bytes = out_ws, ws, wb.value
    cabi.check(dev.L.grl_gqa_decode(dev.h, C.byref(p)))
    p.out, p.workspace, p.workspace_bytes = out_st, None, 0        # no workspace from the caller
    cabi.check(dev.L.grl_gqa_decode_static(dev.h, C.byref(p)))
    dev.sync()
    a = dev.download(out_ws, q.shape, np.float32)
    b = dev.download(out_st, q.shape, np.float32)
    for x in (qd, out_ws, out_st, ws):
        dev.free(x)
    return a, b


def test_static_scratch_decode_matches_workspace_decode():
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    from oracle import attention_oracle as orc
    dev = cabi.Device(0)
    try:
        rng = np.random.default_rng(31)
        B, Hq, Hkv, D = 4, 32, 8, 128
        # first call: long sequences, many splits -> the array is filled with partials
        pc1 = PagedCache(dev, B, Hkv, D, 2048, dtype=cabi.BF16)
        k1 = rng.standard_normal((B, 2000, Hkv, D), dtype=np.float32)
        v1 = rng.standard_normal((B, 2000, Hkv, D), dtype=np.float32)
        pc1.append(k1, v1)
        q1 = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
        a, b = _decode_both(dev, pc1, q1, 8)
        np.testing.assert_allclose(b, a, atol=1e-6, rtol=0)
        want = orc.gqa_decode_attention(q1, orc.round_bf16(k1), orc.round_bf16(v1), Hq, Hkv, D)
        assert np.abs(b - want).max() <= 5e-3
        # second call right after: other data, shorter sequences, fewer splits, fp32 cache (the other kernel);
        # whatever the first call left in the array must not show
        pc2 = PagedCache(dev, 2, 2, 64, 256, page_tokens=16, dtype=cabi.F32)
        k2 = rng.standard_normal((2, 100, 2, 64), dtype=np.float32)
        v2 = rng.standard_normal((2, 100, 2, 64), dtype=np.float32)
        pc2.append(k2, v2)
        q2 = rng.standard_normal((2, 1, 4, 64), dtype=np.float32)
        a2, b2 = _decode_both(dev, pc2, q2, 3)
        np.testing.assert_allclose(b2, a2, atol=1e-6, rtol=0)
        np.testing.assert_allclose(b2, orc.gqa_decode_attention(q2, k2, v2, 4, 2, 64), atol=1e-4, rtol=0)
        # a request beyond the built-in 4 MiB is refused with a message, and nothing is launched
        p = cabi.DecodeParams()
        p.kv = pc1.layout()
        qd, od = dev.upload(q1), dev.malloc(q1.nbytes)
        p.q, p.out, p.num_q_heads, p.n_splits, p.max_seq_len = qd, od, Hq, 256, 2000
        launches = dev.L.grl_launch_count()
        rc = dev.L.grl_gqa_decode_static(dev.h, C.byref(p))
        assert rc == -1 and b"built-in array" in dev.L.grl_last_error()
        assert dev.L.grl_launch_count() == launches
    finally:
        dev.close()

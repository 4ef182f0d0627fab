"""Quantised KV storage on the paged cache (FP8-E4M3 keys, INT4 values, float16 group scales) against the
oracle's restatement of the reference's quantiser (cpp/src/ops/kv_cache.cpp:272-399, :500-577): the stored
bytes bit for bit, the dequantised cache bit for bit, attention over it within the fp32 kernel's tolerance."""
import ctypes as C

import numpy as np
import pytest

from gpu_helpers import quant_v_offsets

pytestmark = pytest.mark.gpu


def _stored(dev, pc, b, T):
    """Bytes of sequence b, token-major: (keys (T,H,D) u8, values (T,H,D/2) u8, scales (T,H,D/32) u16)."""
    H, D, P = pc.Hkv, pc.D, pc.P
    rows = pc.max_pages * pc.B * H * P
    kq = dev.download(pc.k_pages, (rows, D), np.uint8)
    vq = dev.download(pc.v_pages, (rows // P, P * D // 2), np.uint8)       # one row per (page, kv head) block
    sc = dev.download(pc.scales, (rows, D // 32), np.uint16)
    idx = np.array([[(pc.table_host[b, t // P] * H + h) * P + t % P for h in range(H)] for t in range(T)])
    off = quant_v_offsets(P, D)                                           # where the library keeps each value byte
    vals = np.array([[vq[(pc.table_host[b, t // P] * H + h), off[t % P]] for h in range(H)] for t in range(T)])
    assert len(np.unique(off)) == off.size and off.max() == off.size - 1  # a permutation of the block's bytes
    return kq[idx], vals, sc[idx]


@pytest.mark.parametrize("D,P,T", [(128, 64, 150), (64, 16, 37), (32, 64, 5)])
def test_quantised_append_gather_match_the_oracle_bit_for_bit(D, P, T):
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    from oracle import c_oracle
    dev = cabi.Device(0)
    try:
        rng = np.random.default_rng(11)
        B, H = 2, 3
        k = rng.standard_normal((B, T, H, D), dtype=np.float32)
        v = rng.standard_normal((B, T, H, D), dtype=np.float32)
        # magnitudes that exercise every branch of the encoder: an all-zero group, tiny values (code 0),
        # values below 1 after scaling (the truncated-exponent quirk), one dominant element
        k[0, 0, 0, :32] = 0.0
        k[0, 1, 1, :16] *= 1e-4
        k[1, 2, 2, 5] = 250.0
        v[0, 0, 0, :32] = 0.0
        v[1, 1, 0, 7] = -40.0
        pc = PagedCache(dev, B, H, D, T + 9, page_tokens=P, dtype=cabi.FP8_INT4, shuffle_pages=True, seed=3)
        pc.append(k[:, :T // 2], v[:, :T // 2])             # two appends: the second starts inside a page
        pc.append(k[:, T // 2:], v[:, T // 2:])
        for b in range(B):
            want = c_oracle.kv_quantize(k[b], v[b])
            got = _stored(dev, pc, b, T)
            for name, g, w in zip(("keys", "values", "scales"), got, want):
                assert np.array_equal(g, w), f"{name} of sequence {b}: {np.argwhere(g != w)[:5]}"
            gk, gv = pc.gather(b)
            wk, wv = c_oracle.kv_dequantize(*want)
            assert np.array_equal(gk.view(np.uint32), wk.view(np.uint32))
            assert np.array_equal(gv.view(np.uint32), wv.view(np.uint32))
    finally:
        dev.close()


def _dequantised(k, v):
    from oracle import c_oracle
    kd = np.stack([c_oracle.kv_dequantize(*c_oracle.kv_quantize(k[b], v[b]))[0] for b in range(k.shape[0])])
    vd = np.stack([c_oracle.kv_dequantize(*c_oracle.kv_quantize(k[b], v[b]))[1] for b in range(k.shape[0])])
    return kd, vd


def test_decode_over_the_quantised_cache():
    """The generic kernel dequantises with the reference's float32 arithmetic: 2e-4 of the oracle on the same cache."""
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    from oracle import attention_oracle as orc
    dev = cabi.Device(0)
    try:
        rng = np.random.default_rng(12)
        B, Hq, Hkv, D, T = 2, 8, 2, 128, 777
        k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
        v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
        q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
        pc = PagedCache(dev, B, Hkv, D, 832, dtype=cabi.FP8_INT4)
        pc.append(k, v)
        kd, vd = _dequantised(k, v)
        want = orc.gqa_decode_attention(q, kd, vd, Hq, Hkv, D)
        for splits in (1, 5):
            got = pc.decode(q, n_splits=splits, force_simt=True)
            assert np.abs(got - want).max() <= 2e-4, splits
    finally:
        dev.close()


@pytest.mark.parametrize("Hq,Hkv,lens,P", [(8, 2, (777, 64), 64), (8, 8, (130, 1), 64), (16, 2, (1000, 999), 64),
                                           (3, 1, (65, 447), 64), (32, 8, (4352, 4100), 64), (8, 2, (777, 49), 16),
                                           (16, 4, (1000, 33), 32)])
def test_tensor_core_decode_over_the_quantised_cache(Hq, Hkv, lens, P):
    """head_dim 128 with pages of 64, 32 or 16 tokens runs on the tensor-core kernel (q and P rounded to float16, the cache
    dequantised in registers): 1e-3 of the output's scale against the oracle on the same quantised cache, for unsplit,
    split and kernel-chosen launches, ragged lengths and scattered pages; and it is the kernel that ran."""
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    from oracle import attention_oracle as orc
    dev = cabi.Device(0)
    try:
        rng = np.random.default_rng(Hq * 100 + Hkv)
        B, D, T = len(lens), 128, max(lens)
        k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32) * rng.uniform(0.2, 3.0, (B, T, Hkv, 1)).astype(np.float32)
        v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
        q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
        pc = PagedCache(dev, B, Hkv, D, T + 64, page_tokens=P, dtype=cabi.FP8_INT4, shuffle_pages=True, seed=5)
        pc.append(k, v)
        cut = np.array(lens, np.int32)                      # shorten the sequences: the pages keep their tails
        dev.L.grl_memcpy_h2d(dev.h, pc.seq_lens, cut.ctypes.data_as(C.c_void_p), cut.nbytes)
        dev.sync()
        pc.lens[:] = cut
        kd, vd = _dequantised(k, v)
        want = np.concatenate([orc.gqa_decode_attention(q[b:b + 1], kd[b:b + 1, :lens[b]], vd[b:b + 1, :lens[b]], Hq, Hkv, D)
                               for b in range(B)])
        tol = 1e-3 * np.abs(want).max()
        before = dev.L.grl_launch_count()
        for splits in (1, 0, 3):
            got = pc.decode(q, n_splits=splits)
            assert np.abs(got - want).max() <= tol, (splits, np.abs(got - want).max(), tol)
        assert dev.L.grl_launch_count() - before == 3        # one launch each: the kernel merges its own splits
        simt = pc.decode(q, n_splits=2, force_simt=True)
        assert np.abs(simt - want).max() <= tol
    finally:
        dev.close()


def test_quantised_append_with_rope_and_queries():
    """RoPE of the new keys happens before the quantiser; the step's queries are rotated alongside."""
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    from oracle import attention_oracle as orc, c_oracle
    dev = cabi.Device(0)
    try:
        rng = np.random.default_rng(13)
        B, Hq, Hkv, D, T = 1, 4, 2, 64, 40
        k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
        v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
        q = rng.standard_normal((B, T, Hq, D), dtype=np.float32)
        pc = PagedCache(dev, B, Hkv, D, 64, page_tokens=16, dtype=cabi.FP8_INT4)
        q_rot = pc.append(k, v, q=q, rope_mode=cabi.ROPE_INTERLEAVED)
        pos = np.arange(T)
        k_rot = orc.rope_interleaved(k.transpose(0, 2, 1, 3), pos).transpose(0, 2, 1, 3)
        np.testing.assert_allclose(q_rot, orc.rope_interleaved(q.transpose(0, 2, 1, 3), pos).transpose(0, 2, 1, 3), atol=2e-6)
        wk, wv = c_oracle.kv_dequantize(*c_oracle.kv_quantize(k_rot[0], v[0]))
        gk, gv = pc.gather(0)
        # the rotation differs in the last bit here and there, which may move a key across a code boundary
        assert np.mean(gk != wk) < 0.01 and np.abs(gk - wk).max() <= 0.13 * np.abs(wk).max()
        assert np.array_equal(gv, wv)
        assert (dev.download(pc.seq_lens, (B,), np.int32) == T).all()
    finally:
        dev.close()


def test_python_ops_on_a_quantised_cache():
    """create_kv_cache(use_asymmetric_quant=True): append, kv_cache_decode (dequantised, bit for bit) and decode."""
    import grilly_core
    from oracle import attention_oracle as orc, c_oracle
    ctx = grilly_core.Device()
    rng = np.random.default_rng(14)
    Hq, Hkv, D, T = 8, 2, 64, 90
    kv = grilly_core.create_kv_cache(ctx, num_heads=Hkv, head_dim=D, compression_ratio=1, max_cache_tokens=128,
                                     use_asymmetric_quant=True, use_h2o=False, page_tokens=16)
    k = rng.standard_normal((T, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((T, Hkv, D), dtype=np.float32)
    grilly_core.kv_cache_append(ctx, kv, k[:50], v[:50])
    grilly_core.kv_cache_append(ctx, kv, k[50:], v[50:])
    assert kv.current_len == T
    got = grilly_core.kv_cache_decode(ctx, kv)
    wk, wv = c_oracle.kv_dequantize(*c_oracle.kv_quantize(k, v))
    assert np.array_equal(got["keys"], wk) and np.array_equal(got["values"], wv)
    q = rng.standard_normal((1, 1, Hq, D), dtype=np.float32)
    out = grilly_core.gqa_attention(ctx, q, kv)
    want = orc.gqa_decode_attention(q, wk[None], wv[None], Hq, Hkv, D)
    assert np.abs(out - want).max() <= 2e-4
    assert abs(kv.stats()["compression_ratio"] - 8.0 / 1.5) < 1e-3     # the reference's figure: scales not counted
    with pytest.raises(RuntimeError, match="quantised"):
        grilly_core.kv_cache_compact(ctx, kv)
    grilly_core.destroy_kv_cache(ctx, kv)

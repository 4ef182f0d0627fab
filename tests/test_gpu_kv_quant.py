"""Quantised KV storage on the paged cache (FP8-E4M3 keys, INT4 values, float16 group scales) against the
oracle's restatement of the reference's quantiser (cpp/src/ops/kv_cache.cpp:272-399, :500-577): the stored
bytes bit for bit, the dequantised cache bit for bit, attention over it within the fp32 kernel's tolerance."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _stored(dev, pc, b, T):
    """Bytes of sequence b, token-major: (keys (T,H,D) u8, values (T,H,D/2) u8, scales (T,H,D/32) u16)."""
    H, D, P = pc.Hkv, pc.D, pc.P
    rows = pc.max_pages * pc.B * H * P
    kq = dev.download(pc.k_pages, (rows, D), np.uint8)
    vq = dev.download(pc.v_pages, (rows, D // 2), np.uint8)
    sc = dev.download(pc.scales, (rows, D // 32), np.uint16)
    idx = np.array([[(pc.table_host[b, t // P] * H + h) * P + t % P for h in range(H)] for t in range(T)])
    return kq[idx], vq[idx], sc[idx]


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


def test_decode_over_the_quantised_cache():
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    from oracle import attention_oracle as orc, c_oracle
    dev = cabi.Device(0)
    try:
        rng = np.random.default_rng(12)
        B, Hq, Hkv, D, T = 2, 8, 2, 128, 777
        k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
        v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
        q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
        pc = PagedCache(dev, B, Hkv, D, 832, dtype=cabi.FP8_INT4)
        pc.append(k, v)
        kd = np.stack([c_oracle.kv_dequantize(*c_oracle.kv_quantize(k[b], v[b]))[0] for b in range(B)])
        vd = np.stack([c_oracle.kv_dequantize(*c_oracle.kv_quantize(k[b], v[b]))[1] for b in range(B)])
        want = orc.gqa_decode_attention(q, kd, vd, Hq, Hkv, D)
        for splits in (1, 5):
            got = pc.decode(q, n_splits=splits)
            assert np.abs(got - want).max() <= 2e-4, splits
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

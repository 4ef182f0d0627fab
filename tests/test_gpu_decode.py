"""GPU parity of the decode path: paged KV append / gather, GQA decode, LSE merge, RoPE and
attention-mask ops, against the oracle and the golden vectors."""
import ctypes as C
import os

import numpy as np
import pytest

import cases
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu

TOL_TC = 5e-3   # tensor-core decode against the oracle on the same bf16 cache
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_golden.npz"))


@pytest.fixture(scope="module")
def dev():
    from grilly_next import cabi
    d = cabi.Device(0)
    yield d
    d.close()


@pytest.fixture(scope="module")
def gpu():
    from grilly_next import Compute
    g = Compute()
    yield g
    g.cleanup()


@pytest.mark.parametrize("name", list(cases.DECODE_CASES))
def test_gqa_decode_fp32_cache_matches_golden(gpu, name):
    c = cases.DECODE_CASES[name]
    q, k, v = cases.decode_inputs(c)
    out = gpu.gqa_attention(q, k, v)               # explicit (B,T,Hkv,D) arrays, fp32 storage
    assert out.shape == q.shape
    tol = 1e-5 if c["scale"] < 1 else 1e-4
    np.testing.assert_allclose(out, GOLD[f"decode/{name}"], atol=tol, rtol=0)


@pytest.mark.parametrize("name", ["gqa_t300", "gqa_t4097", "mha_t130"])
def test_gqa_decode_bf16_cache(gpu, name):
    c = cases.DECODE_CASES[name]
    q, k, v = cases.decode_inputs(c)
    out = gpu.gqa_attention(q, k, v, dtype="bf16")
    assert np.abs(out - GOLD[f"decode/{name}"]).max() <= 2e-2
    # against the oracle evaluated on the bf16-rounded cache the kernel is much tighter: what is left
    # is the bf16 rounding of the probabilities on the tensor-core path (head_dim 128 and 64, 64-token pages)
    want = orc.gqa_decode_attention(q, orc.round_bf16(k), orc.round_bf16(v), c["Hq"], c["Hkv"], c["D"])
    assert np.abs(out - want).max() <= TOL_TC


def test_cache_len_argument_and_split_counts(gpu, dev):
    from gpu_helpers import PagedCache
    c = cases.DECODE_CASES["gqa_t4097"]
    q, k, v = cases.decode_inputs(c)
    out = gpu.gqa_attention(q, k, v, cache_len=1000)
    want = orc.gqa_decode_attention(q, k, v, c["Hq"], c["Hkv"], c["D"], cache_len=1000)
    np.testing.assert_allclose(out, want, atol=1e-4, rtol=0)
    # every split count gives the same answer, including more splits than pages
    from grilly_next import cabi
    pc = PagedCache(dev, c["B"], c["Hkv"], c["D"], 4200, dtype=cabi.F32, shuffle_pages=True, seed=3)
    pc.append(k, v)
    base = None
    for ns in (1, 2, 3, 8, 64, 128):
        o = pc.decode(q, n_splits=ns)
        np.testing.assert_allclose(o, GOLD["decode/gqa_t4097"], atol=1e-4, rtol=0)
        base = o if base is None else base
        assert np.abs(o - base).max() <= 2e-5
    auto = pc.decode(q)
    assert pc.last_splits >= 1
    np.testing.assert_allclose(auto, GOLD["decode/gqa_t4097"], atol=1e-4, rtol=0)


def test_ragged_batch_and_empty_sequence(dev):
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    rng = np.random.default_rng(11)
    B, Hq, Hkv, D = 3, 8, 2, 64
    pc = PagedCache(dev, B, Hkv, D, 512, page_tokens=16, dtype=cabi.F32)
    lens = [0, 37, 130]
    model = orc.PagedKVModel(B, Hkv, D, 16, dtype="fp32")
    # grow the sequences by different amounts: append one sequence at a time through a length-1 batch view
    Tmax = max(lens)
    k = rng.standard_normal((B, Tmax, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, Tmax, Hkv, D), dtype=np.float32)
    for b in range(B):
        if lens[b]:
            model.append(b, k[b, :lens[b]], v[b, :lens[b]])
    # device: write lengths directly, then append nothing more -- emulate by appending Tmax and resetting seq_lens
    pc.append(k, v)
    cabi.check(dev.L.grl_memcpy_h2d(dev.h, pc.seq_lens, np.asarray(lens, np.int32).ctypes.data_as(C.c_void_p), 4 * B))
    dev.sync()
    pc.lens[:] = lens
    q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
    out = pc.decode(q, n_splits=4)
    Kd, Vd, L = model.dense()
    want = np.zeros_like(q)
    for b in range(B):
        if lens[b]:
            want[b] = orc.gqa_decode_attention(q[b:b + 1], Kd[b:b + 1], Vd[b:b + 1], Hq, Hkv, D, cache_len=lens[b])[0]
    np.testing.assert_allclose(out, want, atol=1e-4, rtol=0)
    assert np.all(out[0] == 0), "an empty sequence attends to nothing and yields zeros"


def test_append_gather_roundtrip_is_bit_exact(dev):
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    rng = np.random.default_rng(12)
    B, Hkv, D = 2, 3, 128
    for dtype, name in ((cabi.BF16, "bf16"), (cabi.F32, "fp32")):
        pc = PagedCache(dev, B, Hkv, D, 300, page_tokens=64, dtype=dtype, shuffle_pages=True, seed=5)
        model = orc.PagedKVModel(B, Hkv, D, 64, dtype=name)
        for n in (1, 62, 1, 1, 130, 3):          # crosses page boundaries at 64, 128, 192
            k = rng.standard_normal((B, n, Hkv, D), dtype=np.float32)
            v = rng.standard_normal((B, n, Hkv, D), dtype=np.float32)
            pc.append(k, v)
            for b in range(B):
                model.append(b, k[b], v[b])
        for b in range(B):
            gk, gv = pc.gather(b)
            mk, mv = model.gather(b)
            assert gk.shape == mk.shape == (198, Hkv, D)
            assert np.array_equal(gk.view(np.uint32), mk.view(np.uint32))
            assert np.array_equal(gv.view(np.uint32), mv.view(np.uint32))


def test_append_with_rope_and_pos_base(dev):
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    rng = np.random.default_rng(13)
    B, Hq, Hkv, D = 2, 4, 2, 64
    pc = PagedCache(dev, B, Hkv, D, 256, dtype=cabi.F32)
    k0 = rng.standard_normal((B, 70, Hkv, D), dtype=np.float32)
    v0 = rng.standard_normal((B, 70, Hkv, D), dtype=np.float32)
    pc.append(k0, v0, rope_mode=cabi.ROPE_INTERLEAVED, pos_base=1000)
    gk, gv = pc.gather(1)
    want_k = orc.rope_interleaved(k0[1].transpose(1, 0, 2), 1000 + np.arange(70)).transpose(1, 0, 2)
    np.testing.assert_allclose(gk, want_k, atol=2e-6, rtol=0)
    assert np.array_equal(gv, v0[1])
    # one more token with q: both rotated at position 1000 + 70
    k1 = rng.standard_normal((B, 1, Hkv, D), dtype=np.float32)
    v1 = rng.standard_normal((B, 1, Hkv, D), dtype=np.float32)
    q1 = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
    qr = pc.append(k1, v1, q=q1, rope_mode=cabi.ROPE_HALF, theta=500.0, pos_base=1000)
    want_q = orc.rope_half(q1, 500.0, positions=[1070])
    np.testing.assert_allclose(qr, want_q, atol=2e-6, rtol=0)
    gk, _ = pc.gather(0)
    np.testing.assert_allclose(gk[70:71], orc.rope_half(k1[0:1], 500.0, positions=[1070])[0], atol=2e-6, rtol=0)
    # angles stay accurate at large positions (double-precision range reduction)
    pc2 = PagedCache(dev, 1, 1, 128, 64, dtype=cabi.F32)
    kk = rng.standard_normal((1, 1, 1, 128), dtype=np.float32)
    pc2.append(kk, kk, rope_mode=cabi.ROPE_INTERLEAVED, pos_base=131071)
    gk, _ = pc2.gather(0)
    np.testing.assert_allclose(gk[0, 0], orc.rope_interleaved(kk[0, 0], [131071])[0], atol=4e-6, rtol=0)


def test_decode_step_loop_matches_oracle(gpu):
    """KVCache + decode_step through the Python ops: prefill a cache, then several steps with RoPE,
    compared step by step with the oracle on the same (bf16-rounded) cache contents."""
    rng = np.random.default_rng(14)
    B, Hq, Hkv, D, T0, steps = 3, 8, 2, 128, 100, 5
    kv = gpu.create_kv_cache(num_heads=Hkv, head_dim=D, compression_ratio=1, max_cache_tokens=256, use_h2o=False,
                             batch_size=B, page_tokens=64, dtype="bf16")
    k0 = rng.standard_normal((B, T0, Hkv, D), dtype=np.float32)
    v0 = rng.standard_normal((B, T0, Hkv, D), dtype=np.float32)
    gpu.kv_cache_append(kv, k0, v0, rope_theta=10000.0)
    assert kv.current_len == T0
    model = orc.PagedKVModel(B, Hkv, D, 64, dtype="bf16")
    for b in range(B):
        model.append(b, orc.rope_interleaved(k0[b].transpose(1, 0, 2), np.arange(T0)).transpose(1, 0, 2), v0[b])
    for t in range(steps):
        q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
        k1 = rng.standard_normal((B, 1, Hkv, D), dtype=np.float32)
        v1 = rng.standard_normal((B, 1, Hkv, D), dtype=np.float32)
        out = gpu.decode_step(kv, q, k1, v1, rope_theta=10000.0)
        pos = [T0 + t]
        for b in range(B):
            model.append(b, orc.rope_interleaved(k1[b].transpose(1, 0, 2), pos).transpose(1, 0, 2), v1[b])
        Kd, Vd, L = model.dense()
        qr = orc.rope_interleaved(q.transpose(0, 2, 1, 3), pos).transpose(0, 2, 1, 3)
        want = orc.gqa_decode_attention(qr, Kd, Vd, Hq, Hkv, D)
        assert np.abs(out - want).max() <= TOL_TC, f"step {t}"
    assert kv.current_len == T0 + steps
    dec = gpu.kv_cache_decode(kv, seq=2)
    mk, mv = model.gather(2)
    assert np.array_equal(dec["keys"], mk) and np.array_equal(dec["values"], mv)
    st = kv.stats()
    assert st["current_tokens"] == T0 + steps and st["total_appended"] == B * (T0 + steps)
    assert {"current_tokens", "max_tokens", "total_evicted", "total_appended", "compression_ratio",
            "avg_attention_score"} <= set(st)
    gpu.destroy_kv_cache(kv)
    with pytest.raises(RuntimeError):
        gpu.kv_cache_decode(kv)


def test_kv_cache_reference_single_sequence_form(gpu):
    # the reference call shape: create_kv_cache(...) then append (n, heads, head_dim) arrays
    rng = np.random.default_rng(15)
    kv = gpu.create_kv_cache(max_seq_len=128, num_heads=4, head_dim=64, compression_ratio=1, max_cache_tokens=128,
                             use_h2o=False, dtype="fp32")
    k = rng.standard_normal((10, 4, 64), dtype=np.float32)
    v = rng.standard_normal((10, 4, 64), dtype=np.float32)
    gpu.kv_cache_append(kv, k, v)
    gpu.kv_cache_append(kv, k[:3], v[:3])
    assert kv.current_len == 13
    d = gpu.kv_cache_decode(kv)
    assert d["keys"].shape == (13, 4, 64)
    assert np.array_equal(d["keys"], np.concatenate([k, k[:3]])) and np.array_equal(d["values"], np.concatenate([v, v[:3]]))
    with pytest.raises(RuntimeError, match="max_cache_tokens"):
        gpu.kv_cache_append(kv, np.zeros((200, 4, 64), np.float32), np.zeros((200, 4, 64), np.float32))
    mla = gpu.create_kv_cache()                   # the reference default: MLA latents, ratio 4 (tests/test_mla_latent_path.py)
    assert mla.stats()["compression_ratio"] == 8.0
    gpu.destroy_kv_cache(mla)
    # the eviction calls of the reference API: a quarter of the 13 tokens goes (all scores are zero, so the
    # tie rule picks the first three), compaction closes the gaps
    gpu.kv_cache_evict_h2o(kv)
    assert gpu.kv_cache_token_meta(kv)["tombstone"].tolist() == [1, 1, 1] + [0] * 10
    gpu.kv_cache_compact(kv)
    assert kv.current_len == 10
    assert np.array_equal(gpu.kv_cache_decode(kv)["keys"], np.concatenate([k, k[:3]])[3:])


def test_lse_merge_matches_oracle(dev):
    from grilly_next import cabi
    rng = np.random.default_rng(16)
    rows, D, P = 10, 128, 5
    o = rng.standard_normal((P, rows, D)).astype(np.float32)
    m = (rng.standard_normal((P, rows)) * 4).astype(np.float32)
    l = (rng.random((P, rows)) * 50 + 0.1).astype(np.float32)
    m[2, :] = -1e30; l[2, :] = 0; o[2] = 0            # an empty part
    parts = np.concatenate([o.reshape(P, -1), m, l], axis=1).astype(np.float32)
    pd = dev.upload(parts)
    od = dev.malloc(rows * (D + 2) * 4)
    cabi.check(dev.L.grl_lse_merge(dev.h, pd, P, parts.shape[1], rows, D, 1, od))
    got = dev.download(od, (rows, D), np.float32)
    np.testing.assert_allclose(got, orc.lse_merge(o, m, l), atol=1e-5, rtol=1e-5)
    # un-normalised combination, merged again with itself = same result (what the cross-GPU stage relies on)
    cabi.check(dev.L.grl_lse_merge(dev.h, pd, P, parts.shape[1], rows, D, 0, od))
    comb = dev.download(od, (rows * (D + 2),), np.float32)
    np.testing.assert_allclose(comb[:rows * D].reshape(rows, D) / comb[rows * D + rows:][:, None],
                               orc.lse_merge(o, m, l), atol=1e-5, rtol=1e-5)


def test_partial_outputs_merge_across_shards(dev):
    """KV split in contiguous shards (the layout of the multi-GPU long-context decode): per-shard
    partials merged by grl_lse_merge equal the unsharded result."""
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    rng = np.random.default_rng(17)
    B, Hq, Hkv, D, T, G = 1, 32, 8, 128, 1024, 4
    q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
    k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    parts = []
    for g in range(G):
        pc = PagedCache(dev, B, Hkv, D, T // G, dtype=cabi.BF16)
        pc.append(k[:, g * T // G:(g + 1) * T // G], v[:, g * T // G:(g + 1) * T // G])
        parts.append(pc.decode(q, partial=True))
    rows = B * Hq
    pd = dev.upload(np.stack(parts))
    od = dev.malloc(rows * D * 4)
    cabi.check(dev.L.grl_lse_merge(dev.h, pd, G, rows * (D + 2), rows, D, 1, od))
    got = dev.download(od, (B, 1, Hq, D), np.float32)
    want = orc.gqa_decode_attention(q, orc.round_bf16(k), orc.round_bf16(v), Hq, Hkv, D)
    assert np.abs(got - want).max() <= TOL_TC


@pytest.mark.parametrize("D,Hq,Hkv,P", [(128, 16, 4, 64), (64, 12, 4, 64), (64, 8, 1, 64), (128, 16, 4, 16), (128, 8, 2, 32),
                                        (64, 12, 4, 16)])
def test_tensor_core_and_simt_decode_agree(dev, D, Hq, Hkv, P):
    """Same bf16 paged cache through both decode kernels: ragged lengths, shuffled pages, a partial
    last page, every split count; the SIMT kernel is the tight one, the tensor-core kernel must stay
    within the rounding of its bf16 probabilities."""
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    rng = np.random.default_rng(21)
    B = 3
    lens = [1000, 65, 517]
    pc = PagedCache(dev, B, Hkv, D, 1024, page_tokens=P, dtype=cabi.BF16, shuffle_pages=True, seed=9)
    k = rng.standard_normal((B, 1000, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, 1000, Hkv, D), dtype=np.float32)
    pc.append(k, v)
    cabi.check(dev.L.grl_memcpy_h2d(dev.h, pc.seq_lens, np.asarray(lens, np.int32).ctypes.data_as(C.c_void_p), 4 * B))
    dev.sync()
    pc.lens[:] = lens
    # poison the tail of the last page of sequence 1 in V with NaN: rows past the length must not leak
    q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
    want = np.zeros_like(q)
    for b in range(B):
        want[b] = orc.gqa_decode_attention(q[b:b + 1], orc.round_bf16(k[b:b + 1]), orc.round_bf16(v[b:b + 1]), Hq, Hkv, D,
                                           cache_len=lens[b])[0]
    for ns in (1, 2, 5, 16):
        simt = pc.decode(q, n_splits=ns, force_simt=True)
        tc = pc.decode(q, n_splits=ns)
        assert np.abs(simt - want).max() <= 2e-4
        assert np.abs(tc - want).max() <= TOL_TC
        assert np.all(np.isfinite(tc))
        assert np.abs(tc - simt).max() > 0          # two different kernels ran


def test_rope_op(gpu):
    rng = np.random.default_rng(18)
    x = rng.standard_normal((2, 50, 3, 64), dtype=np.float32)
    np.testing.assert_allclose(gpu.rope(x), orc.rope_half(x), atol=2e-6, rtol=0)
    np.testing.assert_allclose(gpu.rope(x, base=500.0, scaling=4.0), orc.rope_half(x, 500.0, 4.0), atol=2e-6, rtol=0)
    th = np.arange(64)[:, None] * orc.rope_inv_freq(64, 10000.0)[None]
    cos, sin = np.cos(th).astype(np.float32), np.sin(th).astype(np.float32)
    np.testing.assert_allclose(gpu.rope(x, cos=cos, sin=sin), orc.rope_half(x, cos=cos, sin=sin), atol=2e-6, rtol=0)
    yi = gpu.rope(x, mode="interleaved")
    want = orc.rope_interleaved(x.transpose(0, 2, 1, 3), np.arange(50)).transpose(0, 2, 1, 3)
    np.testing.assert_allclose(yi, want, atol=2e-6, rtol=0)
    with pytest.raises(RuntimeError):
        gpu.rope(x[0])


def test_attention_mask_op(gpu):
    rng = np.random.default_rng(19)
    s = rng.standard_normal((2, 3, 33, 33), dtype=np.float32)
    assert np.array_equal(gpu.attention_mask(s, causal=True), orc.attention_mask(s, causal=True))
    km = (rng.random((2, 33)) > 0.4).astype(np.float32)
    assert np.array_equal(gpu.attention_mask(s, mask=km, mask_value=-7.5), orc.attention_mask(s, mask=km, mask_value=-7.5))
    with pytest.raises(RuntimeError):
        gpu.attention_mask(s)

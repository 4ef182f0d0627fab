"""GPU parity of the eviction family on the paged cache (C ABI and Python module) against the oracle.
Everything here is exact: scores add in the reference's order, selection and row moves are index work."""
import ctypes as C

import numpy as np
import pytest

from oracle import attention_oracle as orc
from oracle import kv_evict_oracle as ev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from grilly_next import cabi
    d = cabi.Device(0)
    yield d
    d.close()


class Meta:
    def __init__(self, dev, pc):
        from grilly_next import cabi
        self.dev, self.B = dev, pc.B
        self.cap = pc.max_pages * pc.P
        n = self.B * self.cap
        self.cum, self.tomb, self.rel, self.evicted = dev.malloc(n * 4), dev.malloc(n), dev.malloc(n * 4), dev.malloc(self.B * 4)
        for p, nb in ((self.cum, n * 4), (self.tomb, n), (self.rel, n * 4), (self.evicted, self.B * 4)):
            cabi.check(dev.L.grl_memset(dev.h, p, 0, nb))
        dev.sync()
        m = cabi.KVMeta()
        m.cum_score, m.tombstone, m.relevance, m.evicted, m.capacity = self.cum, self.tomb, self.rel, self.evicted, self.cap
        self.m = m

    def host(self):
        d = self.dev
        return (d.download(self.cum, (self.B, self.cap), np.float32), d.download(self.tomb, (self.B, self.cap), np.uint8),
                d.download(self.rel, (self.B, self.cap), np.float32), d.download(self.evicted, (self.B,), np.int32))


def _set_lens(dev, pc, lens):
    from grilly_next import cabi
    arr = np.asarray(lens, np.int32)
    cabi.check(dev.L.grl_memcpy_h2d(dev.h, pc.seq_lens, arr.ctypes.data_as(C.c_void_p), arr.nbytes))
    dev.sync()
    pc.lens[:] = arr


@pytest.mark.parametrize("dtype_name,D", [("bf16", 128), ("fp32", 64), ("bf16", 32)])
def test_evict_and_compact_through_the_c_abi(dev, dtype_name, D):
    from grilly_next import cabi
    from gpu_helpers import PagedCache
    dtype = cabi.BF16 if dtype_name == "bf16" else cabi.F32
    rng = np.random.default_rng(11)
    B, Hkv, T = 3, 2, 300
    lens = [300, 131, 64]
    pc = PagedCache(dev, B, Hkv, D, 320, dtype=dtype, shuffle_pages=True, seed=3)
    k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    pc.append(k, v)
    _set_lens(dev, pc, lens)
    stored = (lambda x: orc.round_bf16(x)) if dtype == cabi.BF16 else (lambda x: x)
    meta = Meta(dev, pc)
    l = pc.layout()
    # ---- scores: two rounds of column sums, 7 and 300 query rows
    want_cum = [np.zeros(n, np.float32) for n in lens]
    for q_rows in (7, 300):
        attn = rng.random((B, q_rows, T), dtype=np.float32)
        ad = dev.upload(attn)
        cabi.check(dev.L.grl_kv_score_accumulate(dev.h, C.byref(l), C.byref(meta.m), ad, q_rows, T))
        dev.sync(); dev.free(ad)
        for b, n in enumerate(lens):
            want_cum[b] = ev.accumulate_scores(want_cum[b], attn[b][:, :n])
    cum, tomb, _, _ = meta.host()
    for b, n in enumerate(lens):
        assert np.array_equal(cum[b, :n], want_cum[b]) and not cum[b, n:].any()
    # make some ties so that the tie rule is exercised
    cum[0, [5, 17, 200]] = cum[0, 3]
    cabi.check(dev.L.grl_memcpy_h2d(dev.h, meta.cum, cum.ctypes.data_as(C.c_void_p), cum.nbytes)); dev.sync()
    want_cum = [cum[b, :n].copy() for b, n in enumerate(lens)]
    # ---- H2O selection: explicit count (larger than the shortest sequence: that one is left alone), then default
    want_tomb = [np.zeros(n, np.uint8) for n in lens]
    for num in (70, 0):
        cabi.check(dev.L.grl_kv_evict_lowest(dev.h, C.byref(l), C.byref(meta.m), num)); dev.sync()
        for b in range(B):
            _, want_tomb[b] = ev.evict_h2o(want_cum[b], want_tomb[b], None, num)
    _, tomb, _, _ = meta.host()
    for b, n in enumerate(lens):
        assert np.array_equal(tomb[b, :n], want_tomb[b]), f"sequence {b}"
    assert want_tomb[2].sum() == 16                       # 70 >= 64: only the default quarter applied
    # ---- heuristic on top
    cabi.check(dev.L.grl_kv_evict_heuristic(dev.h, C.byref(l), C.byref(meta.m), C.c_float(0.35))); dev.sync()
    want_rel = []
    for b in range(B):
        want_tomb[b], r = ev.evict_heuristic(want_cum[b], want_tomb[b], 0.35)
        want_rel.append(r)
    _, tomb, rel, _ = meta.host()
    for b, n in enumerate(lens):
        assert np.array_equal(tomb[b, :n], want_tomb[b]) and np.array_equal(rel[b, :n], want_rel[b])
    # ---- compaction
    nb = C.c_size_t()
    cabi.check(dev.L.grl_kv_compact_scratch_bytes(C.byref(l), C.byref(meta.m), C.byref(nb)))
    scratch = dev.malloc(nb.value)
    cabi.check(dev.L.grl_kv_compact(dev.h, C.byref(l), C.byref(meta.m), scratch, nb.value)); dev.sync()
    new_lens = dev.download(pc.seq_lens, (B,), np.int32)
    cum, tomb, _, evicted = meta.host()
    pc.lens[:] = new_lens
    for b, n in enumerate(lens):
        wk, wv, wc = ev.compact(stored(k[b, :n]), stored(v[b, :n]), want_cum[b], want_tomb[b])
        assert new_lens[b] == len(wc) and evicted[b] == n - len(wc)
        gk, gv = pc.gather(b)
        assert np.array_equal(gk, wk) and np.array_equal(gv, wv)
        assert np.array_equal(cum[b, :len(wc)], wc) and not cum[b, len(wc):].any() and not tomb[b].any()
    # compaction with nothing to remove leaves everything in place
    cabi.check(dev.L.grl_kv_compact(dev.h, C.byref(l), C.byref(meta.m), scratch, nb.value)); dev.sync()
    assert np.array_equal(dev.download(pc.seq_lens, (B,), np.int32), new_lens)
    # ---- the next append rotates its keys at the true position: evicted + length
    k1 = rng.standard_normal((B, 1, Hkv, D), dtype=np.float32)
    pc.append(k1, k1, rope_mode=cabi.ROPE_INTERLEAVED, pos_offsets=meta.evicted)
    for b in range(B):
        gk, _ = pc.gather(b)
        pos = np.array([int(evicted[b]) + int(new_lens[b])])
        want = stored(orc.rope_interleaved(k1[b:b + 1].transpose(0, 2, 1, 3), pos)[0].transpose(1, 0, 2)[0])
        assert np.abs(gk[-1] - want).max() <= (1e-2 if dtype == cabi.BF16 else 1e-5)
    dev.free(scratch)


def test_reference_api_flow():
    import grilly_core as core
    ctx = core.Device()
    rng = np.random.default_rng(5)
    H, D, T = 4, 64, 96
    kv = core.create_kv_cache(ctx, max_seq_len=128, num_heads=H, head_dim=D, compression_ratio=1, max_cache_tokens=128,
                              use_h2o=True, eviction_threshold=0.2, dtype="fp32")
    k = rng.standard_normal((T, H, D), dtype=np.float32)
    v = rng.standard_normal((T, H, D), dtype=np.float32)
    core.kv_cache_append(ctx, kv, k, v)
    attn = rng.random((T, T), dtype=np.float32)
    core.kv_cache_evict_h2o(ctx, kv, attn, 10)
    want_cum, want_tomb = ev.evict_h2o(np.zeros(T, np.float32), np.zeros(T, np.uint8), attn, 10)
    meta = core.kv_cache_token_meta(ctx, kv)
    assert np.array_equal(meta["cumulative_score"], want_cum) and np.array_equal(meta["tombstone"], want_tomb)
    assert abs(kv.stats()["avg_attention_score"] - ev.average_score(want_cum, want_tomb)) < 1e-6
    core.kv_cache_evict_speculative(ctx, kv)
    want_tomb, want_rel = ev.evict_heuristic(want_cum, want_tomb, 0.2)
    meta = core.kv_cache_token_meta(ctx, kv)
    assert np.array_equal(meta["tombstone"], want_tomb) and np.array_equal(meta["predicted_relevance"], want_rel)
    core.kv_cache_compact(ctx, kv)
    wk, wv, wc = ev.compact(k, v, want_cum, want_tomb)
    assert kv.current_len == len(wc) and kv.stats()["total_evicted"] == T - len(wc)
    d = core.kv_cache_decode(ctx, kv)
    assert np.array_equal(d["keys"], wk) and np.array_equal(d["values"], wv)
    # appending past max_cache_tokens evicts the lowest-scoring tokens first (kv_cache.cpp:161-172)
    n_now = kv.current_len
    extra = 128 - n_now + 5
    k2 = rng.standard_normal((extra, H, D), dtype=np.float32)
    core.kv_cache_append(ctx, kv, k2, k2)
    assert kv.current_len == 128
    _, t2 = ev.evict_h2o(wc, np.zeros(len(wc), np.uint8), None, 5)
    wk2, _, _ = ev.compact(wk, wv, wc, t2)
    d = core.kv_cache_decode(ctx, kv)
    assert np.array_equal(d["keys"], np.concatenate([wk2, k2]))
    with pytest.raises(RuntimeError, match="attention_scores must be"):
        core.kv_cache_evict_h2o(ctx, kv, np.zeros((3, 3), np.float32))
    core.destroy_kv_cache(ctx, kv)


def test_decode_after_compaction_matches_oracle():
    import grilly_core as core
    ctx = core.Device()
    rng = np.random.default_rng(6)
    B, Hq, Hkv, D, T = 2, 8, 2, 128, 200
    kv = core.create_kv_cache(ctx, max_seq_len=256, num_heads=Hkv, head_dim=D, compression_ratio=1, max_cache_tokens=256,
                              batch_size=B)
    k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    core.kv_cache_append(ctx, kv, k, v)
    attn = rng.random((B, T, T), dtype=np.float32)
    core.kv_cache_evict_h2o(ctx, kv, attn, 50)
    core.kv_cache_compact(ctx, kv)
    assert kv.seq_lens == [150, 150]
    q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
    out = core.gqa_attention(ctx, q, kv)
    for b in range(B):
        cum, tomb = ev.evict_h2o(np.zeros(T, np.float32), np.zeros(T, np.uint8), attn[b], 50)
        wk, wv, _ = ev.compact(orc.round_bf16(k[b]), orc.round_bf16(v[b]), cum, tomb)
        want = orc.gqa_decode_attention(q[b:b + 1], wk[None], wv[None], Hq, Hkv, D)
        assert np.abs(out[b:b + 1] - want).max() <= 5e-3
    core.destroy_kv_cache(ctx, kv)


@pytest.mark.parametrize("dtype,D,tol", [("bf16", 128, 2e-3), ("fp32", 64, 1e-5), ("bf16", 64, 2e-3)])
def test_decode_accumulates_attention_mass(dtype, D, tol):
    # tensor-core kernel (bf16, D=128) and the generic kernel: the scores the step computed become the
    # cumulative H2O scores, summed over the query heads, without an attention matrix from the caller
    import grilly_core as core
    ctx = core.Device()
    rng = np.random.default_rng(8)
    B, Hq, Hkv, T = 2, 8, 2, 333
    kv = core.create_kv_cache(ctx, max_seq_len=512, num_heads=Hkv, head_dim=D, compression_ratio=1, max_cache_tokens=512,
                              batch_size=B, dtype=dtype)
    k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    core.kv_cache_append(ctx, kv, k, v)
    ks = orc.round_bf16(k) if dtype == "bf16" else k
    want_cum = np.zeros((B, T), np.float64)
    for step in range(2):
        q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
        plain = core.gqa_attention(ctx, q, kv)
        out = core.gqa_attention(ctx, q, kv, accumulate_scores=True)
        assert np.abs(out - plain).max() <= 1e-5
        for b in range(B):
            for h in range(Hq):
                s = ks[b, :, h // (Hq // Hkv), :].astype(np.float64) @ q[b, 0, h].astype(np.float64) / np.sqrt(D)
                p = np.exp(s - s.max())
                want_cum[b] += p / p.sum()
        for b in range(B):
            got = core.kv_cache_token_meta(ctx, kv, b)["cumulative_score"]
            assert np.abs(got - want_cum[b]).max() <= tol * (step + 1)
            assert abs(got.sum() - Hq * (step + 1)) <= 1e-2        # every head hands out one unit of mass per step
    # the decode-step form appends first, so the new token receives mass too
    q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
    kn = rng.standard_normal((B, 1, Hkv, D), dtype=np.float32)
    core.decode_step(ctx, kv, q, kn, kn, rope_theta=0.0, accumulate_scores=True)
    got = core.kv_cache_token_meta(ctx, kv, 0)["cumulative_score"]
    assert got.shape == (T + 1,) and got[-1] > 0 and abs(got.sum() - 3 * Hq) <= 2e-2
    core.destroy_kv_cache(ctx, kv)


def test_eviction_head_training_and_prediction():
    # kv_cache_init_eviction_head / kv_cache_train_eviction_head / kv_cache_evict_speculative with a trained head
    import grilly_core as core
    ctx = core.Device()
    rng = np.random.default_rng(9)
    H, D, T, inp, hid = 2, 64, 150, 24, 16
    kv = core.create_kv_cache(ctx, max_seq_len=256, num_heads=H, head_dim=D, compression_ratio=1, max_cache_tokens=256,
                              eviction_threshold=0.45, dtype="fp32")
    k = rng.standard_normal((T, H, D), dtype=np.float32)
    core.kv_cache_append(ctx, kv, k, k)
    feats = rng.standard_normal((T, inp), dtype=np.float32)
    # before a head exists (or before its first update) the call is the heuristic, as in the reference
    core.kv_cache_train_eviction_head(ctx, kv, feats, np.ones((3, T), np.float32), 3)      # no head: a no-op
    core.kv_cache_init_eviction_head(ctx, kv, inp, hid, 0.5)
    w = core.kv_cache_eviction_head_weights(ctx, kv)
    lim1, lim2 = np.sqrt(6.0 / (inp + hid)), np.sqrt(6.0 / (hid + 1))
    assert w["w1"].shape == (inp, hid) and np.abs(w["w1"]).max() <= lim1 and np.abs(w["w2"]).max() <= lim2
    assert not w["b1"].any() and not w["b2"].any() and w["total_updates"] == 0 and w["w1"].std() > 0.1 * lim1
    # some tombstones first (they are skipped by training and prediction)
    core.kv_cache_evict_h2o(ctx, kv, rng.random((T, T), dtype=np.float32), 20)
    tomb = core.kv_cache_token_meta(ctx, kv)["tombstone"]
    params = (w["w1"], w["b1"], w["w2"], w["b2"])
    for step in range(3):
        attn = rng.random((11, T), dtype=np.float32)
        core.kv_cache_train_eviction_head(ctx, kv, feats, attn, 11)
        *params, rel = ev.head_train_step(*params, feats, attn, tomb, 0.5)
        got = core.kv_cache_eviction_head_weights(ctx, kv)
        for name, want in zip(("w1", "b1", "w2", "b2"), params):
            assert np.abs(got[name] - want).max() <= 2e-6, (step, name)
        assert got["total_updates"] == step + 1
        assert np.abs(core.kv_cache_token_meta(ctx, kv)["predicted_relevance"] - rel).max() <= 2e-6
    # prediction with the trained head tombstones what falls below the threshold
    core.kv_cache_evict_speculative(ctx, kv, feats)
    want_tomb, want_rel = ev.head_predict(*params, feats, tomb, 0.45)
    meta = core.kv_cache_token_meta(ctx, kv)
    near = np.abs(want_rel - 0.45) < 1e-5                         # predictions on the threshold may fall either way
    assert np.array_equal(meta["tombstone"][~near], want_tomb[~near])
    assert np.abs(meta["predicted_relevance"] - want_rel).max() <= 2e-6
    assert want_tomb.sum() > tomb.sum()
    with pytest.raises(RuntimeError, match="hidden_states must be"):
        core.kv_cache_evict_speculative(ctx, kv, feats[:, :5])
    core.destroy_kv_cache(ctx, kv)


def test_swizzle_kv():
    import grilly_core as core
    ctx = core.Device()
    rng = np.random.default_rng(10)
    for shape, wave in (((2, 3, 100, 64), 32), ((1, 2, 64, 128), 32), ((1, 1, 7, 5), 4)):
        x = rng.standard_normal(shape, dtype=np.float32)
        got = core.swizzle_kv(ctx, x, wave_size=wave)
        assert got.ndim == 1 and np.array_equal(got, ev.swizzle(x, wave))
    x = rng.standard_normal((2, 2, 64, 64), dtype=np.float32)
    back = core.swizzle_kv(ctx, core.swizzle_kv(ctx, x).reshape(x.shape), reverse=True)
    assert np.array_equal(back, x)
    with pytest.raises(RuntimeError, match="multiples of wave_size"):
        core.swizzle_kv(ctx, np.zeros((1, 1, 10, 64), np.float32), reverse=True)
    with pytest.raises(RuntimeError, match="input must be 4D"):
        core.swizzle_kv(ctx, np.zeros((4, 4), np.float32))

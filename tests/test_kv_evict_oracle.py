"""The eviction oracle against a literal transcription of the reference's loops (small cases, CPU)."""
import numpy as np

from oracle import kv_evict_oracle as ev


def _reference_loops_h2o(cum, tomb, attn, num_evict):
    # cpp/src/ops/kv_cache.cpp:595-634 statement by statement
    cum, tomb = cum.copy(), tomb.copy()
    n = len(cum)
    if num_evict == 0:
        num_evict = n // 4
    if num_evict >= n:
        return cum, tomb
    if attn is not None:
        for t in range(n):
            total = np.float32(0.0)
            for q in range(n):
                total = np.float32(total + attn[q, t])
            cum[t] = np.float32(cum[t] + total)
    idx = sorted(range(n), key=lambda i: (cum[i], i))      # partial_sort by score; ties by index
    for i in range(num_evict):
        tomb[idx[i]] = 1
    return cum, tomb


def test_h2o_matches_the_loops():
    rng = np.random.default_rng(0)
    for n, k in ((16, 0), (16, 5), (33, 8), (8, 8), (8, 20), (5, 0)):
        cum = rng.random(n, dtype=np.float32)
        cum[rng.integers(0, n, 3)] = cum[0]                # ties
        tomb = np.zeros(n, np.uint8)
        attn = rng.random((n, n), dtype=np.float32)
        for a in (None, attn):
            want = _reference_loops_h2o(cum, tomb, a, k)
            got = ev.evict_h2o(cum, tomb, a, k)
            assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


def test_compact_and_average():
    rng = np.random.default_rng(1)
    T, H, D = 12, 2, 4
    k = rng.standard_normal((T, H, D), dtype=np.float32)
    v = rng.standard_normal((T, H, D), dtype=np.float32)
    cum = rng.random(T, dtype=np.float32)
    tomb = np.zeros(T, np.uint8)
    tomb[[0, 3, 4, 11]] = 1
    k2, v2, c2 = ev.compact(k, v, cum, tomb)
    keep = [1, 2, 5, 6, 7, 8, 9, 10]
    assert np.array_equal(k2, k[keep]) and np.array_equal(v2, v[keep]) and np.array_equal(c2, cum[keep])
    assert abs(ev.average_score(cum, tomb) - float(cum[keep].astype(np.float64).mean())) < 1e-6
    assert ev.average_score(cum, np.ones(T, np.uint8)) == 0.0


def test_heuristic_threshold():
    cum = np.array([0.0, 4.0, 1.0, 2.0], np.float32)
    tomb = np.array([0, 0, 1, 0], np.uint8)
    t2, rel = ev.evict_heuristic(cum, tomb, 0.3)
    # relevance: 0.7*cum/4 + 0.3*t/4 -> [0, 0.775, -, 0.575]; token 0 falls below 0.3, token 2 stays tombstoned
    assert t2.tolist() == [1, 0, 1, 0]
    assert np.allclose(rel, [0.0, 0.775, 0.0, 0.575], atol=1e-6)
    # all-zero scores: the inverse maximum is 1 (kv_cache.cpp:913)
    t3, rel3 = ev.evict_heuristic(np.zeros(4, np.float32), np.zeros(4, np.uint8), 0.1)
    assert t3.tolist() == [1, 1, 0, 0] and np.allclose(rel3, [0, 0.075, 0.15, 0.225], atol=1e-6)


def test_head_training_lowers_the_loss():
    # the restated SGD step is a gradient step of the binary cross-entropy it claims to minimise
    rng = np.random.default_rng(2)
    T, inp, hid = 40, 6, 5
    w1 = rng.standard_normal((inp, hid)).astype(np.float32) * 0.5
    b1, w2, b2 = np.zeros(hid, np.float32), rng.standard_normal(hid).astype(np.float32) * 0.5, np.zeros(1, np.float32)
    feats = rng.standard_normal((T, inp)).astype(np.float32)
    attn = rng.random((7, T), dtype=np.float32)
    tomb = np.zeros(T, np.uint8); tomb[3] = 1
    received = attn.sum(0)
    labels = (received > np.sort(received)[T // 2]).astype(np.float64)

    def loss(params):
        total = 0.0
        for t in range(T):
            if tomb[t]:
                continue
            _, s = ev._head_forward(*params, feats[t])
            s = min(max(float(s), 1e-7), 1 - 1e-7)
            total += -(labels[t] * np.log(s) + (1 - labels[t]) * np.log(1 - s))
        return total

    params = (w1, b1, w2, b2)
    before = loss(params)
    for _ in range(20):
        *params, rel = ev.head_train_step(*params, feats, attn, tomb, lr=0.5)
    assert loss(params) < before and rel[3] == 0.0 and np.all((rel >= 0) & (rel <= 1))
    t2, r2 = ev.head_predict(*params, feats, tomb, 0.5)
    assert t2[3] == 1 and np.array_equal(t2[r2 < 0.5] == 1, np.ones((r2 < 0.5).sum(), bool))


def test_swizzle_matches_the_index_formula():
    # destination index of cpp/src/ops/swizzle.cpp:77-84, element by element
    rng = np.random.default_rng(3)
    B, H, S, D, W = 2, 3, 10, 6, 4
    x = rng.standard_normal((B, H, S, D), dtype=np.float32)
    sp, dp = 12, 8
    want = np.zeros(B * H * sp * dp, np.float32)
    for b in range(B):
        for h in range(H):
            for s in range(S):
                for d in range(D):
                    dst = (b * H + h) * sp * dp + (s // W) * ((dp // W) * W * W) + (d // W) * W * W + (s % W) * W + d % W
                    want[dst] = x[b, h, s, d]
    got = ev.swizzle(x, W)
    assert np.array_equal(got, want)
    assert np.array_equal(ev.unswizzle(got, x.shape, W), x)

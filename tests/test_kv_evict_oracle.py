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

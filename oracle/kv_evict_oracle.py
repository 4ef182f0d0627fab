"""CPU restatement of the reference's KV-cache eviction family.  TEST INFRASTRUCTURE ONLY: the
product never imports this module.

Follows cpp/src/ops/kv_cache.cpp of the reference: kvCacheEvictH2O (:595-634), the untrained-head
branch of kvCacheEvictSpeculative (:905-929), kvCacheCompact (:941-992) and the score average of
kvCacheGetStats (:1004-1015).  The reference keeps one TokenMeta per token (cumulativeScore,
predictedRelevance, nextActive with UINT32_MAX-1 as the tombstone); here those are plain arrays.

Parity unpinned: the reference has no test or golden vector for these functions (its library cannot be
built here either), so this file is a restatement of the source, checked only against a literal
loop-by-loop transcription of the same source on small cases (tests/test_kv_evict_oracle.py).

One choice the reference leaves open is made here: std::partial_sort does not order equal scores, so
"the numEvict lowest" is ambiguous under ties; ties go to the lowest index.
"""
import numpy as np


def accumulate_scores(cum, attn):
    """cum[t] += sum_q attn[q, t], the sum taken in ascending q in float32 (kv_cache.cpp:606-615)."""
    cum = np.asarray(cum, np.float32).copy()
    attn = np.asarray(attn, np.float32)
    total = np.zeros(attn.shape[1], np.float32)
    for q in range(attn.shape[0]):
        total = total + attn[q]
    cum[: attn.shape[1]] = cum[: attn.shape[1]] + total
    return cum


def evict_h2o(cum, tomb, attn=None, num_evict=0):
    """Returns (cum, tomb) after kvCacheEvictH2O on a sequence of len(cum) tokens."""
    cum = np.asarray(cum, np.float32).copy()
    tomb = np.asarray(tomb, np.uint8).copy()
    n = len(cum)
    k = num_evict if num_evict else n // 4          # :598-600
    if k >= n:                                      # :601 -- before the scores are touched
        return cum, tomb
    if attn is not None:
        cum = accumulate_scores(cum, attn)
    order = np.argsort(cum, kind="stable")          # lowest first, ties by index
    tomb[order[:k]] = 1                             # :630-633 (already tombstoned tokens take part, as there)
    return cum, tomb


def evict_heuristic(cum, tomb, threshold):
    """Returns (tomb, relevance) after the fallback branch of kvCacheEvictSpeculative."""
    cum = np.asarray(cum, np.float32)
    tomb = np.asarray(tomb, np.uint8).copy()
    n = len(cum)
    rel = np.zeros(n, np.float32)
    mx = np.float32(0.0)
    for t in range(n):                              # :906-911: every token, tombstoned or not
        if cum[t] > mx:
            mx = cum[t]
    inv = np.float32(1.0) / mx if mx > 0 else np.float32(1.0)
    for t in range(n):
        if tomb[t]:
            continue
        norm = np.float32(cum[t] * inv)
        rec = np.float32(np.float32(t) / np.float32(n))
        rel[t] = np.float32(np.float32(0.7) * norm) + np.float32(np.float32(0.3) * rec)
        if rel[t] < np.float32(threshold):
            tomb[t] = 1
    return tomb, rel


def compact(keys, values, cum, tomb):
    """keys/values (T, H, D).  Returns (keys, values, cum) of the live tokens in their old order
    (kv_cache.cpp:946-991)."""
    live = np.flatnonzero(np.asarray(tomb) == 0)
    return keys[live], values[live], np.asarray(cum, np.float32)[live]


def average_score(cum, tomb):
    """kvCacheGetStats: mean cumulative score of the active tokens, summed in index order in float32."""
    total, active = np.float32(0.0), 0
    for t in range(len(cum)):
        if not tomb[t]:
            total = np.float32(total + np.float32(cum[t]))
            active += 1
    return float(total / np.float32(active)) if active else 0.0

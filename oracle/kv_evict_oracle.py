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


# ---- trainable eviction head (kv_cache.cpp:734-845 and :863-903) -----------------------------------

def _head_forward(w1, b1, w2, b2, x):
    """hidden = relu(W1^T x + b1) with the sum over inputs in ascending order starting from the bias,
    logit = b2 + sum_h w2[h] hidden[h] in ascending h, score = sigmoid(logit): float32 throughout."""
    hidden = b1.astype(np.float32).copy()
    for i in range(w1.shape[0]):
        hidden = hidden + np.float32(x[i]) * w1[i]          # one multiply, one add per term (no fusing)
    hidden = np.maximum(np.float32(0.0), hidden)
    logit = np.float32(b2[0])
    for h in range(len(hidden)):
        logit = np.float32(logit + np.float32(w2[h] * hidden[h]))
    score = np.float32(1.0) / (np.float32(1.0) + np.exp(-logit, dtype=np.float32))
    return hidden, np.float32(score)


def head_train_step(w1, b1, w2, b2, features, attn, tomb, lr):
    """One call of kvCacheTrainEvictionHead.  features (T, in), attn (seq_len, T), tomb (T,).
    Returns (w1, b1, w2, b2, relevance) with relevance[t] = prediction made before the update
    (0 where the token is tombstoned and skipped)."""
    w1, b1, w2, b2 = (np.asarray(a, np.float32).copy() for a in (w1, b1, w2, b2))
    T = features.shape[0]
    received = np.zeros(T, np.float32)
    for q in range(attn.shape[0]):
        received = received + attn[q].astype(np.float32)
    median = np.sort(received)[T // 2]                      # what nth_element leaves at T/2
    labels = (received > median).astype(np.float32)
    g_w1, g_b1 = np.zeros_like(w1), np.zeros_like(b1)
    g_w2, g_b2 = np.zeros_like(w2), np.float32(0.0)
    rel = np.zeros(T, np.float32)
    for t in range(T):
        if tomb[t]:
            continue
        x = features[t].astype(np.float32)
        hidden, score = _head_forward(w1, b1, w2, b2, x)
        rel[t] = score
        d_logit = np.float32(score - labels[t])
        g_w2 = g_w2 + d_logit * hidden
        g_b2 = np.float32(g_b2 + d_logit)
        d_hidden = np.float32(d_logit) * w2 * (hidden > 0).astype(np.float32)
        g_b1 = g_b1 + d_hidden
        g_w1 = g_w1 + x[:, None] * d_hidden[None, :]
    step = np.float32(lr) / np.float32(T)
    return w1 - step * g_w1, b1 - step * g_b1, w2 - step * g_w2, np.float32(b2 - step * g_b2).reshape(1), rel


def head_predict(w1, b1, w2, b2, features, tomb, threshold):
    """Trained-head branch of kvCacheEvictSpeculative: returns (tomb, relevance)."""
    tomb = np.asarray(tomb, np.uint8).copy()
    rel = np.zeros(features.shape[0], np.float32)
    for t in range(features.shape[0]):
        if tomb[t]:
            continue
        _, rel[t] = _head_forward(w1, b1, w2, b2, features[t].astype(np.float32))
        if rel[t] < np.float32(threshold):
            tomb[t] = 1
    return tomb, rel


# ---- block swizzle (cpp/src/ops/swizzle.cpp:49-123) ------------------------------------------------

def swizzle(x, wave=32):
    """(B,H,S,D) -> flat (B*H*S_pad*D_pad) with layout [b][h][s/W][d/W][s%W][d%W], padding zero."""
    B, H, S, D = x.shape
    sp, dp = -(-S // wave) * wave, -(-D // wave) * wave
    pad = np.zeros((B, H, sp, dp), np.float32)
    pad[:, :, :S, :D] = x
    return pad.reshape(B, H, sp // wave, wave, dp // wave, wave).transpose(0, 1, 2, 4, 3, 5).reshape(-1)


def unswizzle(flat, shape, wave=32):
    B, H, S, D = shape
    sp, dp = -(-S // wave) * wave, -(-D // wave) * wave
    pad = np.asarray(flat, np.float32).reshape(B, H, sp // wave, dp // wave, wave, wave).transpose(0, 1, 2, 4, 3, 5)
    return pad.reshape(B, H, sp, dp)[:, :, :S, :D].copy()

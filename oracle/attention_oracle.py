"""CPU oracle for the attention hot path (TEST INFRASTRUCTURE, never the product path).

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this
module; the CUDA library never routes through it.

Every function restates, in numpy, the arithmetic of one piece of the reference
(Grillcheese-AI/grilly-next); the reference file:line each follows is given in its docstring.
Pinned against golden vectors generated from the reference's own numpy references
(tests/golden/make_golden.py) for prefill attention and GQA decode.  The RoPE, attention-mask
and KV append/gather restatements follow shader source only: the reference holds no test or
golden vector for them, so for those ops parity is unpinned.
"""
from __future__ import annotations

import numpy as np

MASKED_SCORE = -1e9  # tests/test_attention.py:30


# --------------------------------------------------------------------------- bf16 helpers
def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit pattern (uint16), round-to-nearest-even (the rounding of cvt.rn.bf16.f32)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    return r.astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bf16 -> float32."""
    return from_bf16_bits(to_bf16_bits(x)).reshape(np.shape(x))


# --------------------------------------------------------------------------- prefill attention
def attention_4d(Q, K, V, mask=None, scale=None, dtype=np.float32):
    """softmax(Q K^T * scale, masked) V on (batch, heads, seq, dim) tensors.

    Follows tests/test_attention.py:20-35 (_ref_attention_4d): scores are scaled, positions with
    mask <= 0 are REPLACED by -1e9 (not added), softmax is max-subtracted, mask is (B,H,S,S).
    `dtype` lets a test evaluate the same arithmetic in float64.
    """
    Q = np.asarray(Q, dtype=dtype)
    K = np.asarray(K, dtype=dtype)
    V = np.asarray(V, dtype=dtype)
    B, H, S, D = Q.shape
    if scale is None:
        scale = 1.0 / np.sqrt(D)
    out = np.empty((B, H, S, V.shape[-1]), dtype=dtype)
    for b in range(B):
        for h in range(H):
            s = (Q[b, h] @ K[b, h].T) * dtype(scale)
            if mask is not None:
                s = np.where(np.asarray(mask)[b, h] > 0, s, dtype(MASKED_SCORE))
            s = s - s.max(axis=-1, keepdims=True)
            p = np.exp(s)
            p /= p.sum(axis=-1, keepdims=True)
            out[b, h] = p @ V[b, h]
    return out


def causal_length_mask(B, H, S, seq_lens=None, causal=True):
    """(B,H,S,S) keep-mask of ones/zeros: lower triangle, and key index < seq_lens[b]."""
    m = np.ones((S, S), dtype=np.float32)
    if causal:
        m = np.tril(m)
    out = np.broadcast_to(m, (B, H, S, S)).copy()
    if seq_lens is not None:
        for b in range(B):
            out[b, :, :, int(seq_lens[b]):] = 0.0
    return out


def expand_mask(mask, B, H, S):
    """Bring any of the reference's three mask conventions to the (B,H,S,S) keep-mask form.

    (B,S): key-padding mask read as mask[b*S + k] by shaders/flash-attention2.glsl:151-154;
    (B,S,S): the B*S*S floats the host uploads in cpp/src/ops/attention.cpp:63-66;
    (B,1,S,S) / (B,H,S,S): tests/test_attention.py:29-30.  Values > 0 keep.
    """
    mask = np.asarray(mask, dtype=np.float32)
    if mask.ndim == 2:
        return np.broadcast_to(mask[:, None, None, :], (B, H, S, S))
    if mask.ndim == 3:
        return np.broadcast_to(mask[:, None, :, :], (B, H, S, S))
    return np.broadcast_to(mask, (B, H, S, S))


# --------------------------------------------------------------------------- RoPE
def rope_inv_freq(D, base):
    """base^(-2i/D) for i in [0, D/2) (flash-attention2-rope.glsl:74-77, rope.glsl:44-50), float64."""
    i = np.arange(D // 2, dtype=np.float64)
    return np.power(np.float64(base), -2.0 * i / np.float64(D))


def rope_interleaved(x, positions, base=10000.0, scaling=1.0):
    """Rotate pairs (2i, 2i+1) of the last axis; x is (..., S, D), positions is (S,).

    Follows shaders/flash-attention2-rope.glsl:74-88,101-141: theta = pos * base^(-2i/D) / scaling,
    y0 = x0 cos - x1 sin, y1 = x0 sin + x1 cos.  Angles in float64, result float32.
    """
    x = np.asarray(x, dtype=np.float32)
    D = x.shape[-1]
    th = np.asarray(positions, dtype=np.float64)[:, None] * rope_inv_freq(D, base)[None, :] / np.float64(scaling)
    c, s = np.cos(th), np.sin(th)
    x0 = x[..., 0::2].astype(np.float64)
    x1 = x[..., 1::2].astype(np.float64)
    y = np.empty(x.shape, dtype=np.float64)
    y[..., 0::2] = x0 * c - x1 * s
    y[..., 1::2] = x0 * s + x1 * c
    return y.astype(np.float32)


def rope_half(x, base=10000.0, scaling=1.0, cos=None, sin=None, positions=None):
    """rotate_half RoPE on (B, S, H, D): y = x*cos + rotate_half(x)*sin, out of place.

    Follows shaders/rope.glsl:76-125: rotate_half(x) = [-x[D/2:], x[:D/2]], position = seq index
    / scaling, frequency index = d mod D/2, optional (max_seq, D/2) cos/sin tables indexed by the
    sequence index (rope.glsl:109-113).
    """
    x = np.asarray(x, dtype=np.float32)
    B, S, H, D = x.shape
    half = D // 2
    if cos is None:
        pos = np.arange(S, dtype=np.float64) if positions is None else np.asarray(positions, np.float64)
        th = (pos / np.float64(scaling))[:, None] * rope_inv_freq(D, base)[None, :]
        c, s = np.cos(th), np.sin(th)
    else:
        c = np.asarray(cos, dtype=np.float64)[:S]
        s = np.asarray(sin, dtype=np.float64)[:S]
    c = c[None, :, None, :]
    s = s[None, :, None, :]
    lo = x[..., :half].astype(np.float64)
    hi = x[..., half:].astype(np.float64)
    y = np.empty(x.shape, dtype=np.float64)
    y[..., :half] = lo * c - hi * s
    y[..., half:] = hi * c + lo * s
    return y.astype(np.float32)


# --------------------------------------------------------------------------- attention-mask op
def attention_mask(scores, mask=None, causal=False, mask_value=-1e9):
    """In-place style fill on materialised (B,H,S,S) scores; returns a new array.

    Follows shaders/attention-mask.glsl:42-54: causal -> scores[k > q] = mask_value; otherwise a
    (B,S) key mask, scores[..., k] = mask_value where mask[b,k] < 0.5.
    """
    out = np.array(scores, dtype=np.float32, copy=True)
    B, H, S, _ = out.shape
    if causal:
        q = np.arange(S)[:, None]
        k = np.arange(S)[None, :]
        out[:, :, k > q] = np.float32(mask_value)
    else:
        drop = np.asarray(mask, dtype=np.float32) < 0.5  # (B,S)
        out = np.where(drop[:, None, None, :], np.float32(mask_value), out)
    return out


# --------------------------------------------------------------------------- GQA decode
def gqa_decode_attention(query, k_cache, v_cache, num_q_heads, num_kv_heads, head_dim,
                         cache_len=None, scale=None, dtype=np.float32):
    """One decode step: query (B,1,Hq,D) over caches (B,T,Hkv,D); returns (B,1,Hq,D).

    Follows tests/test_inference_ops.py:64-95 (_ref_gqa_decode_attention) and
    shaders/gqa-attention.glsl:52-129: kv_head = q_head // (Hq // Hkv), softmax over the first
    cache_len positions.  cache_len may be an int or a per-batch sequence.
    """
    q = np.asarray(query, dtype=dtype)
    B = q.shape[0]
    if scale is None:
        scale = 1.0 / np.sqrt(head_dim)
    if cache_len is None:
        cache_len = k_cache.shape[1]
    lens = np.broadcast_to(np.asarray(cache_len), (B,))
    g = num_q_heads // num_kv_heads
    q = q.reshape(B, num_q_heads, head_dim)
    out = np.zeros((B, num_q_heads, head_dim), dtype=dtype)
    for b in range(B):
        T = int(lens[b])
        kb = np.asarray(k_cache[b, :T], dtype=dtype)
        vb = np.asarray(v_cache[b, :T], dtype=dtype)
        for kvh in range(num_kv_heads):
            qs = q[b, kvh * g:(kvh + 1) * g]                    # (g, D)
            s = (qs @ kb[:, kvh].T) * dtype(scale)              # (g, T)
            s = s - s.max(axis=-1, keepdims=True)
            p = np.exp(s)
            p /= p.sum(axis=-1, keepdims=True)
            out[b, kvh * g:(kvh + 1) * g] = p @ vb[:, kvh]
    return out.reshape(B, 1, num_q_heads, head_dim)


def lse_merge(o_parts, m_parts, l_parts):
    """Merge split-KV partials. o_parts (P, ..., D) un-normalised sums, m_parts/l_parts (P, ...).

    m = max_i m_i; O = sum_i e^{m_i-m} O_i / sum_i e^{m_i-m} l_i (natural-log domain).
    """
    o = np.asarray(o_parts, dtype=np.float64)
    m = np.asarray(m_parts, dtype=np.float64)
    l = np.asarray(l_parts, dtype=np.float64)
    mm = m.max(axis=0)
    w = np.exp(m - mm[None])
    num = (w[..., None] * o).sum(axis=0)
    den = (w * l).sum(axis=0)
    return (num / den[..., None]).astype(np.float32)


# --------------------------------------------------------------------------- paged KV cache model
class PagedKVModel:
    """Host model of the paged head-major cache: pages [page][Hkv][page_tokens][D], block table
    [B][max_pages].  Storage dtype "bf16" rounds on append like the device kernel.

    Append/gather semantics follow cpp/include/grilly/ops/kv_cache.h:153-177 (append
    (numNew, H, D) rows at currentLen; decode returns (T, H, D) float32).
    """

    def __init__(self, batch, num_kv_heads, head_dim, page_tokens=64, dtype="bf16"):
        self.B, self.H, self.D, self.P = batch, num_kv_heads, head_dim, page_tokens
        self.dtype = dtype
        self.k = [[] for _ in range(batch)]
        self.v = [[] for _ in range(batch)]

    def _store(self, x):
        x = np.asarray(x, dtype=np.float32)
        return round_bf16(x) if self.dtype == "bf16" else x

    def append(self, b, keys, values):
        """keys/values (n, Hkv, D) float32 for sequence b."""
        for t in range(keys.shape[0]):
            self.k[b].append(self._store(keys[t]))
            self.v[b].append(self._store(values[t]))

    def gather(self, b):
        T = len(self.k[b])
        if T == 0:
            z = np.zeros((0, self.H, self.D), np.float32)
            return z, z.copy()
        return np.stack(self.k[b]), np.stack(self.v[b])

    def dense(self):
        """(B, Tmax, Hkv, D) zero-padded arrays + lens, the layout of gqa-attention.glsl:14-22."""
        lens = np.array([len(x) for x in self.k], dtype=np.int32)
        T = int(lens.max()) if len(lens) else 0
        K = np.zeros((self.B, T, self.H, self.D), np.float32)
        V = np.zeros_like(K)
        for b in range(self.B):
            if lens[b]:
                K[b, :lens[b]], V[b, :lens[b]] = self.gather(b)
        return K, V, lens


def prefill_flops(D, lens, causal=True, heads=1):
    """4*D*sum n_pairs, n_pairs = L(L+1)/2 causal or L*L."""
    tot = 0
    for L in lens:
        L = int(L)
        tot += L * (L + 1) // 2 if causal else L * L
    return 4 * D * tot * heads

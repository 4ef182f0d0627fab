"""ctypes loader for oracle/liboracle.so (TEST INFRASTRUCTURE; see attn_oracle.c)."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE, "liboracle.so"])


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        _LIB = ctypes.CDLL(path)
        _LIB.oracle_num_threads.restype = ctypes.c_int
    return _LIB


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def attention(Q, K, V, mask_add=None, scale=0.0, causal=False, seq_lens=None):
    Q = np.ascontiguousarray(Q, np.float32)
    K = np.ascontiguousarray(K, np.float32)
    V = np.ascontiguousarray(V, np.float32)
    B, H, S, D = Q.shape
    T = K.shape[2]
    out = np.empty_like(Q)
    m = None if mask_add is None else np.ascontiguousarray(mask_add, np.float32)
    sl = None if seq_lens is None else np.ascontiguousarray(seq_lens, np.int32)
    lib().oracle_attention_f32(_p(Q), _p(K), _p(V), _p(m), _p(out), B, H, S, T, D,
                               ctypes.c_float(scale), int(bool(causal)), _p(sl))
    return out


def gqa_decode(q, k_cache, v_cache, cache_lens=None, scale=0.0):
    q = np.ascontiguousarray(q, np.float32)
    k_cache = np.ascontiguousarray(k_cache, np.float32)
    v_cache = np.ascontiguousarray(v_cache, np.float32)
    B, _, Hq, D = q.shape
    Tmax, Hkv = k_cache.shape[1], k_cache.shape[2]
    out = np.empty_like(q)
    cl = None if cache_lens is None else np.ascontiguousarray(np.broadcast_to(cache_lens, (B,)), np.int32)
    lib().oracle_gqa_decode_f32(_p(q), _p(k_cache), _p(v_cache), _p(out), B, Hq, Hkv, D, Tmax,
                                _p(cl), ctypes.c_float(scale))
    return out


def rope_interleaved(x, base=10000.0, scaling=1.0):
    """(..., S, D) float32 rotated along S at positions 0..S-1 (the C twin of attention_oracle.rope_interleaved)."""
    x = np.ascontiguousarray(x, np.float32)
    S, D = x.shape[-2], x.shape[-1]
    out = np.empty_like(x)
    lib().oracle_rope_interleaved_f32(_p(x), _p(out), ctypes.c_long(x.size // (S * D)), S, D,
                                      ctypes.c_double(base), ctypes.c_double(scaling))
    return out


def kv_quantize(keys, values):
    """(T,H,D) float32 keys / values -> (keys_q (T,H,D) u8, vals_q (T,H,D/2) u8, scales (T,H,ceil(D/32)) u16):
    the reference's FP8 / INT4 storage bytes (kv_quant_oracle.c)."""
    keys = np.ascontiguousarray(keys, np.float32)
    values = np.ascontiguousarray(values, np.float32)
    T, H, D = keys.shape
    G = (D + 31) // 32
    kq = np.empty((T, H, D), np.uint8)
    vq = np.empty((T, H, D // 2), np.uint8)
    sc = np.empty((T, H, G), np.uint16)
    lib().oracle_kv_quantize(_p(keys), _p(values), T, H, D, _p(kq), _p(vq), _p(sc))
    return kq, vq, sc


def kv_dequantize(keys_q, vals_q, scales):
    keys_q = np.ascontiguousarray(keys_q, np.uint8)
    vals_q = np.ascontiguousarray(vals_q, np.uint8)
    scales = np.ascontiguousarray(scales, np.uint16)
    T, H, D = keys_q.shape
    k = np.empty((T, H, D), np.float32)
    v = np.empty((T, H, D), np.float32)
    lib().oracle_kv_dequantize(_p(keys_q), _p(vals_q), _p(scales), T, H, D, _p(k), _p(v))
    return k, v


def num_threads():
    return lib().oracle_num_threads()

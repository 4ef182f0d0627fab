"""Known-answer checks of the quantised-KV oracle against values worked out by hand from the reference's
source (cpp/src/ops/kv_cache.cpp:272-399 encode, :500-577 decode).  The reference holds no test or vector
for these paths (parity unpinned); these cases pin the restatement to the source's arithmetic, quirks
included."""
import ctypes

import numpy as np

from oracle import c_oracle


def _enc(x):
    L = c_oracle.lib()
    L.oracle_fp8_encode.restype = ctypes.c_uint8
    return L.oracle_fp8_encode(ctypes.c_float(x))


def _dec(c):
    L = c_oracle.lib()
    L.oracle_fp8_decode.restype = ctypes.c_float
    return L.oracle_fp8_decode(ctypes.c_uint8(c))


def test_fp8_codes_follow_the_source():
    # 448 = 1.75 * 2^8: exponent int(log2 448) + 7 = 15, mantissa (448/256 - 1) * 8 = 6
    assert _enc(448.0) == 0x7E and _dec(0x7E) == 448.0
    assert _enc(-448.0) == 0xFE and _enc(1000.0) == 0x7E          # clamped first
    assert _enc(1.0) == (7 << 3) and _dec(7 << 3) == 1.0
    assert _enc(3.0) == ((8 << 3) | 4) and _dec((8 << 3) | 4) == 3.0
    assert _enc(1.0 / 1024.0) == 0                                 # below 1/512: zero
    # mantissa truncates: 1.99 -> 1 + 7/8
    assert _enc(1.99) == ((7 << 3) | 7) and _dec((7 << 3) | 7) == 1.875
    # the quirk: below 1 the exponent is truncated toward zero (one too high), the mantissa fraction is negative
    # and the cast wraps it: 0.3 -> int(log2 0.3) = -1 -> e = 6, (0.3 / 0.5 - 1) * 8 = -3.2 -> int -3 -> 0xFD & 7 = 5
    assert _enc(0.3) == ((6 << 3) | 5)
    assert _dec((6 << 3) | 5) == 0.8125                            # so 0.3 comes back as 0.8125
    assert _dec(0x03) == 3.0 * 2.0 ** -9 and _dec(0x83) == -3.0 * 2.0 ** -9


def test_group_scales_values_and_packing():
    T, H, D = 2, 1, 64
    k = np.zeros((T, H, D), np.float32)
    v = np.zeros((T, H, D), np.float32)
    k[0, 0, 0] = 3.5            # group 0 of token 0: max 3.5 -> scale 128 = 2^7 -> float16 bits 0x5800
    k[0, 0, 1] = -1.75          # -1.75 * 128 = -224 = -1.75 * 2^7: e = 14, mant 6, sign
    k[0, 0, 40] = 0.0           # group 1 all zero: scale 1.0 -> 0x3C00
    v[0, 0, 0], v[0, 0, 1], v[0, 0, 2], v[0, 0, 3] = 7.0, -7.0, 2.5, -2.5     # value scale 1: codes 15, 1, 11 (round half away), 5
    kq, vq, sc = c_oracle.kv_quantize(k, v)
    assert sc[0, 0, 0] == 0x5800 and sc[0, 0, 1] == 0x3C00
    assert kq[0, 0, 0] == 0x7E and kq[0, 0, 1] == (0x80 | (14 << 3) | 6)
    assert vq[0, 0, 0] == (15 | (1 << 4)) and vq[0, 0, 1] == (11 | (5 << 4))
    assert (vq[1] == 0x88).all()                                   # zeros are code 8 in both nibbles
    kd, vd = c_oracle.kv_dequantize(kq, vq, sc)
    assert kd[0, 0, 0] == 3.5 and kd[0, 0, 1] == -1.75
    # decode applies the stored KEY scale to the values too: (15 - 8) / 128, not 7.0
    assert vd[0, 0, 0] == 7.0 / 128.0 and vd[0, 0, 1] == -7.0 / 128.0


def test_scale_bits_truncate_the_mantissa():
    # scale = 448 / 3 = 149.333...: float32 0x43155555 -> half: exponent 134 - 112 = 22, mantissa 0x155555 >> 13 = 0xAA
    k = np.zeros((1, 1, 32), np.float32)
    k[0, 0, 5] = 3.0
    _, _, sc = c_oracle.kv_quantize(k, k)
    assert sc[0, 0, 0] == ((22 << 10) | 0xAA)

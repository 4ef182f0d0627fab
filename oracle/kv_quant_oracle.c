/* CPU oracle for the quantised KV storage -- TEST INFRASTRUCTURE, never the product path.
 *
 * Restates, arithmetic step by arithmetic step, the asymmetric quantisation of the reference's
 * ops::kvCacheAppend (cpp/src/ops/kv_cache.cpp:272-399: FP8-E4M3 keys, INT4 values, one float16
 * scale per group of 32 elements) and the dequantisation of ops::kvCacheDecode
 * (cpp/src/ops/kv_cache.cpp:500-577).  Parity unpinned: the reference holds no test or vector for
 * these paths, so the source is the specification, quirks included:
 *   - the scale is stored as float16 by bit surgery that truncates the mantissa and does not
 *     range-check the exponent (:297-303);
 *   - the key exponent is int(log2(|x|)), i.e. truncated toward zero, so magnitudes below 1 get an
 *     exponent one too high and a NEGATIVE mantissa fraction, which static_cast<uint8_t> then
 *     wraps (:318-325); the cast of a negative float to uint8_t is restated as what x86-64
 *     compilers emit for it (convert to int32 with truncation, keep the low 8 bits);
 *   - only the KEY scales reach the cache (:393-398), and decode uses that one array for keys and
 *     values alike (:513-516, :566-570).
 * Layouts here are token-major like the reference's: keys (T,H,D) bytes, values (T,H,D/2) bytes
 * (two per byte, even element in the low nibble; H*D is even), scales (T,H,D/32) uint16.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static uint16_t scale_to_half_bits(float scale) {           /* kv_cache.cpp:297-303 */
    uint32_t b;
    memcpy(&b, &scale, sizeof(float));
    return (uint16_t)(((b >> 16) & 0x8000u) | (((b >> 23) - 112u) << 10) | ((b >> 13) & 0x03FFu));
}

static float half_bits_to_scale(uint16_t h) {               /* kv_cache.cpp:517-530 */
    uint32_t sign = (h >> 15) & 1u, e = (h >> 10) & 0x1Fu, m = h & 0x03FFu;
    if (e == 0) return ldexpf((float)m, -24);
    uint32_t f = (sign << 31) | ((e + 112u) << 23) | (m << 13);
    float s;
    memcpy(&s, &f, sizeof(float));
    return s;
}

uint8_t oracle_fp8_encode(float scaled) {                    /* kv_cache.cpp:306-327 */
    scaled = fmaxf(-448.0f, fminf(448.0f, scaled));
    int sign = scaled < 0 ? 1 : 0;
    float a = fabsf(scaled);
    if (a < 1.0f / 512.0f) return 0;
    int e = (int)log2f(a);                                   /* truncation toward zero */
    e += 7;
    if (e < 0) e = 0;
    if (e > 15) e = 15;
    float mantissa = a / powf(2.0f, (float)(e - 7)) - 1.0f;
    uint8_t mant = (uint8_t)((uint32_t)(int32_t)(mantissa * 8.0f) & 0xFFu) & 0x07u;
    return (uint8_t)((sign << 7) | (e << 3) | mant);
}

float oracle_fp8_decode(uint8_t c) {                         /* kv_cache.cpp:540-552 */
    int s = (c >> 7) & 1, e = (c >> 3) & 0x0F, m = c & 7;
    float v = e == 0 ? ldexpf((float)m, -9) : ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return s ? -v : v;
}

/* keys, values: (T,H,D) float32.  keys_q (T,H,D) bytes, vals_q (T,H,D/2) bytes, scales (T,H,G) uint16 with
 * G = ceil(D/32): the KEY scales (the value scales are computed, used to quantise, and dropped). */
void oracle_kv_quantize(const float* keys, const float* values, int T, int H, int D, uint8_t* keys_q,
                        uint8_t* vals_q, uint16_t* scales) {
    const int G = (D + 31) / 32;
    memset(vals_q, 0, (size_t)T * H * D / 2);
    for (int t = 0; t < T; ++t)
        for (int h = 0; h < H; ++h) {
            const size_t base = ((size_t)t * H + h) * D;
            for (int g = 0; g < G; ++g) {
                const int g0 = g * 32, g1 = g0 + 32 < D ? g0 + 32 : D;
                float max_abs = 0.0f;
                for (int i = g0; i < g1; ++i) { float v = fabsf(keys[base + i]); if (v > max_abs) max_abs = v; }
                const float scale = max_abs > 0.0f ? 448.0f / max_abs : 1.0f;
                scales[((size_t)t * H + h) * G + g] = scale_to_half_bits(scale);
                for (int i = g0; i < g1; ++i) keys_q[base + i] = oracle_fp8_encode(keys[base + i] * scale);
                /* values: kv_cache.cpp:341-381 */
                max_abs = 0.0f;
                for (int i = g0; i < g1; ++i) { float v = fabsf(values[base + i]); if (v > max_abs) max_abs = v; }
                const float vscale = max_abs > 0.0f ? 7.0f / max_abs : 1.0f;
                for (int i = g0; i < g1; ++i) {
                    int q = (int)roundf(values[base + i] * vscale) + 8;
                    if (q < 0) q = 0;
                    if (q > 15) q = 15;
                    const size_t flat = base + i;
                    if (flat % 2 == 0) vals_q[flat / 2] = (uint8_t)(q & 0x0F);
                    else vals_q[flat / 2] |= (uint8_t)((q & 0x0F) << 4);
                }
            }
        }
}

/* kv_cache.cpp:500-577: both keys and values are multiplied by 1/scale of the stored (key) scale. */
void oracle_kv_dequantize(const uint8_t* keys_q, const uint8_t* vals_q, const uint16_t* scales, int T, int H,
                          int D, float* keys, float* values) {
    const int G = (D + 31) / 32;
    for (int t = 0; t < T; ++t)
        for (int h = 0; h < H; ++h) {
            const size_t base = ((size_t)t * H + h) * D;
            for (int g = 0; g < G; ++g) {
                const float scale = half_bits_to_scale(scales[((size_t)t * H + h) * G + g]);
                const float inv = scale > 0.0f ? 1.0f / scale : 1.0f;
                const int g0 = g * 32, g1 = g0 + 32 < D ? g0 + 32 : D;
                for (int i = g0; i < g1; ++i) {
                    keys[base + i] = oracle_fp8_decode(keys_q[base + i]) * inv;
                    const size_t flat = base + i;
                    const uint8_t packed = vals_q[flat / 2];
                    const int q = flat % 2 == 0 ? (packed & 0x0F) : ((packed >> 4) & 0x0F);
                    values[base + i] = (float)(q - 8) * inv;
                }
            }
        }
}

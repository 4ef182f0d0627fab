/* CPU oracle in C for the attention hot path -- TEST INFRASTRUCTURE, never the product path.
 *
 * Only the tests, the smoke check and the benchmark's CPU-baseline leg load this library.
 * Parity pinned through tests/golden (vectors generated from the reference's numpy references);
 * the reference's C++ library itself cannot be compiled without the Vulkan SDK and VMA.
 *
 * oracle_attention_f32 restates step 2 of the reference's C++ CPU attention,
 * cpp/src/experimental/fused_attention.cpp:298-356 (per (b,h,q): scores = q.k*scale (+ additive
 * mask), max-subtracted softmax, weighted sum of V), made parallel over (b,h,q) with OpenMP and
 * generalised to per-batch K/V in (B,H,T,D) layout, which is what the bound flash_attention2 op
 * receives (cpp/python/bindings.cpp:425-432).
 *
 * oracle_gqa_decode_f32 restates shaders/gqa-attention.glsl:52-129 /
 * tests/test_inference_ops.py:64-95 (kv_head = q_head / (Hq/Hkv), softmax over cache_len).
 *
 * oracle_rope_interleaved_f32 restates the rotation of shaders/flash-attention2-rope.glsl:74-88,101-141
 * (pairs (2i, 2i+1), theta = pos * base^(-2i/D) / scaling) in double arithmetic, like the numpy
 * restatement it is checked against (parity unpinned: the reference holds no vector for RoPE).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Q,out: (B,H,S,D); K,V: (B,H,T,D); mask_add: NULL or additive (B,S,T) as in
 * fused_attention.cpp:324-327; causal!=0 limits keys to k <= q + (T - S); seq_lens NULL or
 * per-batch valid key count (rows q >= seq_lens[b] are written as zeros). */
void oracle_attention_f32(const float* Q, const float* K, const float* V, const float* mask_add,
                          float* out, int B, int H, int S, int T, int D, float scale, int causal,
                          const int32_t* seq_lens) {
    if (scale == 0.0f) scale = 1.0f / sqrtf((float)D); /* fused_attention.cpp:261-263 */
    long rows = (long)B * H * S;
#pragma omp parallel
    {
        float* scores = (float*)malloc(sizeof(float) * (size_t)(T > 0 ? T : 1));
#pragma omp for schedule(dynamic, 16)
        for (long r = 0; r < rows; ++r) {
            int q = (int)(r % S);
            int h = (int)((r / S) % H);
            int b = (int)(r / ((long)S * H));
            const float* qv = Q + (size_t)r * D;
            const float* Kb = K + ((size_t)b * H + h) * (size_t)T * D;
            const float* Vb = V + ((size_t)b * H + h) * (size_t)T * D;
            float* o = out + (size_t)r * D;
            int kend = T;
            if (seq_lens) {
                kend = seq_lens[b] < T ? seq_lens[b] : T;
                if (q >= seq_lens[b]) { memset(o, 0, sizeof(float) * D); continue; }
            }
            if (causal) {
                int lim = q + (T - S) + 1;
                if (lim < kend) kend = lim;
            }
            float mx = -1e30f;
            for (int k = 0; k < kend; ++k) {
                const float* kv = Kb + (size_t)k * D;
                float dot = 0.0f;
                for (int d = 0; d < D; ++d) dot += qv[d] * kv[d];
                float s = dot * scale;
                if (mask_add) s += mask_add[((size_t)b * S + q) * T + k];
                scores[k] = s;
                if (s > mx) mx = s;
            }
            float sum = 0.0f;
            for (int k = 0; k < kend; ++k) { scores[k] = expf(scores[k] - mx); sum += scores[k]; }
            float inv = 1.0f / sum;
            memset(o, 0, sizeof(float) * D);
            for (int k = 0; k < kend; ++k) {
                float w = scores[k] * inv;
                const float* vv = Vb + (size_t)k * D;
                for (int d = 0; d < D; ++d) o[d] += w * vv[d];
            }
        }
        free(scores);
    }
}

/* q,out: (B,1,Hq,D); k_cache,v_cache: (B,Tmax,Hkv,D) token-major (gqa-attention.glsl:14-22);
 * cache_lens: per-batch length (<= Tmax). */
void oracle_gqa_decode_f32(const float* q, const float* k_cache, const float* v_cache, float* out,
                           int B, int Hq, int Hkv, int D, int Tmax, const int32_t* cache_lens,
                           float scale) {
    if (scale == 0.0f) scale = 1.0f / sqrtf((float)D);
    int g = Hq / Hkv;
    long rows = (long)B * Hq;
#pragma omp parallel
    {
        float* scores = (float*)malloc(sizeof(float) * (size_t)(Tmax > 0 ? Tmax : 1));
#pragma omp for schedule(dynamic, 1)
        for (long r = 0; r < rows; ++r) {
            int b = (int)(r / Hq), qh = (int)(r % Hq), kvh = qh / g;
            int T = cache_lens ? cache_lens[b] : Tmax;
            const float* qv = q + (size_t)r * D;
            float* o = out + (size_t)r * D;
            float mx = -1e30f;
            for (int t = 0; t < T; ++t) {
                const float* kv = k_cache + (((size_t)b * Tmax + t) * Hkv + kvh) * D;
                float dot = 0.0f;
                for (int d = 0; d < D; ++d) dot += qv[d] * kv[d];
                scores[t] = dot * scale;
                if (scores[t] > mx) mx = scores[t];
            }
            float sum = 0.0f;
            for (int t = 0; t < T; ++t) { scores[t] = expf(scores[t] - mx); sum += scores[t]; }
            memset(o, 0, sizeof(float) * D);
            float inv = 1.0f / (sum > 1e-30f ? sum : 1e-30f);
            for (int t = 0; t < T; ++t) {
                float w = scores[t] * inv;
                const float* vv = v_cache + (((size_t)b * Tmax + t) * Hkv + kvh) * D;
                for (int d = 0; d < D; ++d) o[d] += w * vv[d];
            }
        }
        free(scores);
    }
}

/* x, y: (rows_outer, S, D), rotated along S (position = index in S) out of place; y may equal x. */
void oracle_rope_interleaved_f32(const float* x, float* y, long rows_outer, int S, int D, double base,
                                 double scaling) {
    int half = D / 2;
    double* inv = (double*)malloc(sizeof(double) * (size_t)(half > 0 ? half : 1));
    for (int i = 0; i < half; ++i) inv[i] = pow(base, -2.0 * (double)i / (double)D);
    long total = rows_outer * S;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < total; ++r) {
        int pos = (int)(r % S);
        const float* xr = x + (size_t)r * D;
        float* yr = y + (size_t)r * D;
        for (int i = 0; i < half; ++i) {
            double th = (double)pos * inv[i] / scaling;
            double c = cos(th), s = sin(th);
            double x0 = xr[2 * i], x1 = xr[2 * i + 1];
            yr[2 * i] = (float)(x0 * c - x1 * s);
            yr[2 * i + 1] = (float)(x0 * s + x1 * c);
        }
    }
    free(inv);
}

// Paged head-major KV cache kernels: fused RoPE + cast + scatter append, and gather back to
// token-major float32.  Replaces ops::kvCacheAppend / ops::kvCacheDecode
// (cpp/src/ops/kv_cache.cpp:155-419, 435-578) for the uncompressed mode, in which the reference
// stores only metadata.
#include "common.cuh"

namespace grl {

struct AppendArgs {
    void* k_pages;
    void* v_pages;
    const int32_t* block_table;
    int32_t* seq_lens;
    const float* k_new;
    const float* v_new;
    const float* q_in;
    float* q_out;
    int B, Hkv, Hq, D, P, max_pages, n_new;
    int rope_mode, pos_base, update_lens;
    const int32_t* pos_offsets;
    int32_t* status;     // device status word: GRL_ERR_INVALID when a sequence has no room for the new tokens
    uint16_t* scales;    // quantised cache only
    int skip_kv;         // rotate the queries only (the quantised append stores K and V with its own kernel)
    RopeFreq freq;
};

// grid (chunks, B).  A work item is (token i, head slot, pair j), head slots being the Hkv key/value
// heads followed by the Hq query heads, so that a one-token decode step spreads its (Hkv+Hq)*D/2
// pairs over the whole CTA instead of walking the heads serially behind dependent loads.  With
// update_lens the grid has ONE chunk per sequence, so that the length read at entry cannot race
// with the write at exit.
template <typename T>
__global__ void __launch_bounds__(1024) kv_append_kernel(AppendArgs a) {
    const int b = blockIdx.y;
    const int half = a.D / 2;
    const int len0 = a.seq_lens[b];
    // A sequence without room for the new tokens is left untouched (no store, no length update): the block
    // table has no page for them.  The op layer checks this on the host; a direct caller of the C ABI gets
    // GRL_ERR_KERNEL from the next grl_sync.
    if (len0 < 0 || len0 + a.n_new > a.max_pages * a.P) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && a.status && atomicCAS(a.status, 0, GRL_ERR_INVALID) == 0) {
            a.status[1] = 4 << 28;
            a.status[2] = b;
            a.status[3] = len0;
        }
        return;
    }
    const int pos_off = a.pos_offsets ? a.pos_offsets[b] : 0;
    T* kp = reinterpret_cast<T*>(a.k_pages);
    T* vp = reinterpret_cast<T*>(a.v_pages);
    const int slots = a.Hkv + (a.q_in ? a.Hq : 0);
    const int items = a.n_new * slots * half;
    // The angle depends on (position, pair) only: a thread whose stride keeps its pair (block size a
    // multiple of D/2, the decode step's case) evaluates the double-precision range reduction once.
    int cached_pos = -1, cached_j = -1;
    float c = 1.f, s = 0.f;
#pragma unroll 2
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < items; idx += gridDim.x * blockDim.x) {
        const int j = idx % half;
        const int hs = (idx / half) % slots;
        const int i = idx / (half * slots);
        const int slot_pos = len0 + i;
        const int rope_pos = a.pos_base + pos_off + slot_pos;
        int d0 = 2 * j, d1 = 2 * j + 1;
        if (a.rope_mode == GRL_ROPE_HALF) { d0 = j; d1 = j + half; }
        if (a.rope_mode != GRL_ROPE_NONE && (slot_pos != cached_pos || j != cached_j)) {
            rope_sincos(rope_pos, a.freq.inv_freq[j], &c, &s);
            cached_pos = slot_pos; cached_j = j;
        }
        if (hs < a.Hkv) {
            if (a.skip_kv) continue;
            const int page = a.block_table[(size_t)b * a.max_pages + slot_pos / a.P];
            const int slot = slot_pos % a.P;
            const size_t src = (((size_t)b * a.n_new + i) * a.Hkv + hs) * a.D;
            const size_t dst = (((size_t)page * a.Hkv + hs) * a.P + slot) * a.D;
            const float k0 = a.k_new[src + d0], k1 = a.k_new[src + d1];
            const float v0 = a.v_new[src + d0], v1 = a.v_new[src + d1];
            store_from_float<T>(kp + dst + d0, k0 * c - k1 * s);
            store_from_float<T>(kp + dst + d1, k0 * s + k1 * c);
            store_from_float<T>(vp + dst + d0, v0);
            store_from_float<T>(vp + dst + d1, v1);
        } else {
            const size_t qo = (((size_t)b * a.n_new + i) * a.Hq + (hs - a.Hkv)) * a.D;
            const float q0 = a.q_in[qo + d0], q1 = a.q_in[qo + d1];
            a.q_out[qo + d0] = q0 * c - q1 * s;
            a.q_out[qo + d1] = q0 * s + q1 * c;
        }
    }
    if (a.update_lens) {  // gridDim.x == 1 here
        __syncthreads();
        if (threadIdx.x == 0) a.seq_lens[b] = len0 + a.n_new;
    }
}

__global__ void advance_lens_kernel(int32_t* seq_lens, int B, int n, int capacity) {
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B && seq_lens[b] >= 0 && seq_lens[b] + n <= capacity) seq_lens[b] += n;   // a full sequence was skipped
}

template <typename T>
__global__ void kv_gather_kernel(const T* __restrict__ kp, const T* __restrict__ vp,
                                 const int32_t* __restrict__ block_table, int b, int n_tokens, int Hkv, int D,
                                 int P, int max_pages, float* __restrict__ out_k, float* __restrict__ out_v) {
    const size_t total = (size_t)n_tokens * Hkv * D;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(idx % D);
        const int h = (int)((idx / D) % Hkv);
        const int t = (int)(idx / ((size_t)D * Hkv));
        const int page = block_table[(size_t)b * max_pages + t / P];
        const size_t src = (((size_t)page * Hkv + h) * P + t % P) * D + d;
        out_k[idx] = load_as_float<T>(kp + src);
        out_v[idx] = load_as_float<T>(vp + src);
    }
}

// Block swizzle of cpp/src/ops/swizzle.cpp:49-123: (B,H,S,D) <-> (B,H,S_pad/W,D_pad/W,W,W), padding zero.
// One thread per element of the swizzled tensor; W consecutive threads touch W consecutive floats on
// both sides.
__global__ void swizzle_kv_kernel(const float* __restrict__ in, float* __restrict__ out, int S, int D, int W,
                                  int s_pad, int d_pad, size_t total, int reverse) {
    const int d_blocks = d_pad / W;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int dw = (int)(idx % W);
        const int sw = (int)((idx / W) % W);
        const int db = (int)((idx / ((size_t)W * W)) % d_blocks);
        const size_t rest = idx / ((size_t)W * W * d_blocks);
        const int sb = (int)(rest % (s_pad / W));
        const size_t bh = rest / (s_pad / W);
        const int s = sb * W + sw, d = db * W + dw;
        const bool inside = s < S && d < D;
        const size_t plain = (bh * S + s) * D + d;
        if (reverse) {
            if (inside) out[plain] = in[idx];
        } else {
            out[idx] = inside ? in[plain] : 0.f;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Quantised storage (GRL_FP8_INT4): the reference's asymmetric quantisation, cpp/src/ops/kv_cache.cpp:272-399,
// byte for byte.  One warp owns one group of 32 elements of one (token, kv head): lane = element, the group
// maximum is a warp reduction, every lane encodes its own key byte and value nibble.
__device__ __forceinline__ uint16_t scale_to_half_bits(float scale) {       // kv_cache.cpp:297-303: bit surgery
    const uint32_t b = __float_as_uint(scale);
    return (uint16_t)(((b >> 16) & 0x8000u) | (((b >> 23) - 112u) << 10) | ((b >> 13) & 0x03FFu));
}
__device__ __forceinline__ float half_bits_to_scale(uint16_t h) {           // kv_cache.cpp:517-530
    const uint32_t sign = (h >> 15) & 1u, e = (h >> 10) & 0x1Fu, m = h & 0x03FFu;
    if (e == 0) return (float)m * 5.9604644775390625e-08f;                  // ldexp(m, -24), exact
    return __uint_as_float((sign << 31) | ((e + 112u) << 23) | (m << 13));
}
// int(log2f(a)) of the reference (kv_cache.cpp:318): the float32 logarithm, truncated toward zero.  The
// logarithm is taken in double and rounded to float, which is what a correctly rounded log2f returns.
__device__ __forceinline__ uint8_t fp8_encode(float scaled) {               // kv_cache.cpp:306-327
    scaled = fmaxf(-448.0f, fminf(448.0f, scaled));
    const int sign = scaled < 0.f ? 1 : 0;
    const float a = fabsf(scaled);
    if (a < 1.0f / 512.0f) return 0;
    int e = (int)(float)log2((double)a);
    e = max(0, min(15, e + 7));
    const float mantissa = __fsub_rn(__fdiv_rn(a, __uint_as_float((uint32_t)(e - 7 + 127) << 23)), 1.0f);
    // a negative fraction (magnitudes below 1, whose exponent came out one too high) wraps like the reference's
    // cast does on x86-64: to int32 with truncation, low 8 bits kept
    const uint8_t mant = (uint8_t)((uint32_t)(int)__fmul_rn(mantissa, 8.0f) & 0xFFu) & 0x07u;
    return (uint8_t)((sign << 7) | (e << 3) | mant);
}
__device__ __forceinline__ float fp8_decode(uint8_t c) {                    // kv_cache.cpp:540-552
    const uint32_t s = (c >> 7) & 1u, e = (c >> 3) & 0x0Fu, m = c & 7u;
    const float v = e == 0 ? (float)m * 0.001953125f                         // m * 2^-9
                           : __uint_as_float(((e - 7u + 127u) << 23) | (m << 20));
    return s ? -v : v;
}

// grid (ceil(n_new*Hkv*G / warps per CTA), B), G = D/32 groups per head.  With one CTA per sequence (a decode step) the
// kernel also rotates the step's queries (q_in != NULL) and advances the length (update_lens): one launch per step.
__global__ void __launch_bounds__(1024) kv_append_quant_kernel(AppendArgs a) {
    const int b = blockIdx.y, lane = threadIdx.x & 31;
    const int G = a.D / 32;
    const int len0 = a.seq_lens[b];
    if (len0 < 0 || len0 + a.n_new > a.max_pages * a.P) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && a.status && atomicCAS(a.status, 0, GRL_ERR_INVALID) == 0) {
            a.status[1] = 4 << 28;
            a.status[2] = b;
            a.status[3] = len0;
        }
        return;
    }
    const int pos_off = a.pos_offsets ? a.pos_offsets[b] : 0;
    const int items = a.n_new * a.Hkv * G;
    const int half = a.D / 2;
    uint8_t* kp = reinterpret_cast<uint8_t*>(a.k_pages);
    uint8_t* vp = reinterpret_cast<uint8_t*>(a.v_pages);
    for (int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); item < items; item += gridDim.x * (blockDim.x >> 5)) {
        const int g = item % G, h = (item / G) % a.Hkv, i = item / (G * a.Hkv);
        const int d = g * 32 + lane;
        const int slot_pos = len0 + i;
        const size_t src = (((size_t)b * a.n_new + i) * a.Hkv + h) * a.D;
        float kx = a.k_new[src + d];
        if (a.rope_mode != GRL_ROPE_NONE) {
            int j, d_other;
            bool first;
            if (a.rope_mode == GRL_ROPE_INTERLEAVED) { j = d >> 1; first = (d & 1) == 0; d_other = d ^ 1; }
            else { j = d % half; first = d < half; d_other = first ? d + half : d - half; }
            float c, s;
            rope_sincos(a.pos_base + pos_off + slot_pos, a.freq.inv_freq[j], &c, &s);
            const float other = a.k_new[src + d_other];
            kx = first ? kx * c - other * s : other * s + kx * c;
        }
        const float vx = a.v_new[src + d];
        float kmax = fabsf(kx), vmax = fabsf(vx);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            kmax = fmaxf(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
            vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
        }
        const float kscale = kmax > 0.f ? __fdiv_rn(448.0f, kmax) : 1.0f;
        const float vscale = vmax > 0.f ? __fdiv_rn(7.0f, vmax) : 1.0f;
        const int page = a.block_table[(size_t)b * a.max_pages + slot_pos / a.P];
        const size_t row = ((size_t)page * a.Hkv + h) * a.P + slot_pos % a.P;
        kp[row * a.D + d] = fp8_encode(__fmul_rn(kx, kscale));
        int q = (int)roundf(__fmul_rn(vx, vscale)) + 8;                       // kv_cache.cpp:363-366
        q = max(0, min(15, q));
        const int q_hi = __shfl_down_sync(0xffffffffu, q, 1);
        if ((lane & 1) == 0)
            vp[((size_t)page * a.Hkv + h) * a.P * half + quant_v_off(slot_pos % a.P, d >> 1, a.D)] =
                (uint8_t)((q & 0x0F) | ((q_hi & 0x0F) << 4));
        if (lane == 0) a.scales[row * G + g] = scale_to_half_bits(kscale);   // the value scale is dropped (:393-398)
    }
    if (a.q_in) {           // the queries of the new positions, rotated like the keys (float32 in, float32 out)
        const int qitems = a.n_new * a.Hq * half;
        for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < qitems; idx += gridDim.x * blockDim.x) {
            const int j = idx % half, h = (idx / half) % a.Hq, i = idx / (half * a.Hq);
            int d0 = 2 * j, d1 = 2 * j + 1;
            if (a.rope_mode == GRL_ROPE_HALF) { d0 = j; d1 = j + half; }
            float c = 1.f, s = 0.f;
            if (a.rope_mode != GRL_ROPE_NONE) rope_sincos(a.pos_base + pos_off + len0 + i, a.freq.inv_freq[j], &c, &s);
            const size_t qo = (((size_t)b * a.n_new + i) * a.Hq + h) * a.D;
            const float q0 = a.q_in[qo + d0], q1 = a.q_in[qo + d1];
            a.q_out[qo + d0] = q0 * c - q1 * s;
            a.q_out[qo + d1] = q0 * s + q1 * c;
        }
    }
    if (a.update_lens) {    // gridDim.x == 1 here: every warp has read len0
        __syncthreads();
        if (threadIdx.x == 0) a.seq_lens[b] = len0 + a.n_new;
    }
}

// Dequantise sequence b as token-major float32 (T, Hkv, D): kv_cache.cpp:500-577.  One thread per element.
__global__ void kv_gather_quant_kernel(const uint8_t* __restrict__ kp, const uint8_t* __restrict__ vp,
                                       const uint16_t* __restrict__ scales, const int32_t* __restrict__ block_table,
                                       int b, int n_tokens, int Hkv, int D, int P, int max_pages,
                                       float* __restrict__ out_k, float* __restrict__ out_v) {
    const size_t total = (size_t)n_tokens * Hkv * D;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(idx % D);
        const int h = (int)((idx / D) % Hkv);
        const int t = (int)(idx / ((size_t)D * Hkv));
        const int page = block_table[(size_t)b * max_pages + t / P];
        const size_t row = ((size_t)page * Hkv + h) * P + t % P;
        const float scale = half_bits_to_scale(scales[row * (D / 32) + d / 32]);
        const float inv = scale > 0.f ? __fdiv_rn(1.0f, scale) : 1.0f;
        out_k[idx] = __fmul_rn(fp8_decode(kp[row * D + d]), inv);
        const uint8_t packed = vp[((size_t)page * Hkv + h) * P * (D / 2) + quant_v_off(t % P, d >> 1, D)];
        const int q = (d & 1) ? (packed >> 4) & 0x0F : packed & 0x0F;
        out_v[idx] = __fmul_rn((float)(q - 8), inv);
    }
}

// C = A B, all row-major float32: the reference's gemm_mnk shader (shaders/gemm_mnk.glsl:34-80), which the MLA
// latent path dispatches (cpp/src/ops/kv_cache.cpp:216-234, :441-498): 16 x 16 tiles in shared memory, the sum
// over k in ascending order with separate multiplies and adds.
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                        float* __restrict__ C, int M, int K, int N) {
    __shared__ float As[16][17], Bs[16][17];
    const int lx = threadIdx.x & 15, ly = threadIdx.x >> 4;
    const int m = blockIdx.y * 16 + ly, n = blockIdx.x * 16 + lx;
    float acc = 0.f;
    for (int k0 = 0; k0 < K; k0 += 16) {
        As[ly][lx] = (m < M && k0 + lx < K) ? A[(size_t)m * K + k0 + lx] : 0.f;
        Bs[ly][lx] = (n < N && k0 + ly < K) ? B[(size_t)(k0 + ly) * N + n] : 0.f;
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) acc = __fadd_rn(acc, __fmul_rn(As[ly][kk], Bs[kk][lx]));
        __syncthreads();
    }
    if (m < M && n < N) C[(size_t)m * N + n] = acc;
}

// rows x [K (D) | V (D)] <-> separate (rows, D) K and V: the concatenation in front of the MLA down-projection
// (kv_cache.cpp:190-203) and the split behind the up-projection (:483-494).
__global__ void mla_concat_kernel(const float* __restrict__ k, const float* __restrict__ v, float* __restrict__ out,
                                  size_t rows, int D) {
    const size_t total = rows * 2 * D;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / (2 * D);
        const int c = (int)(i % (2 * D));
        out[i] = c < D ? k[r * D + c] : v[r * D + c - D];
    }
}
__global__ void mla_split_kernel(const float* __restrict__ in, float* __restrict__ k, float* __restrict__ v,
                                 size_t rows, int D) {
    const size_t total = rows * 2 * D;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / (2 * D);
        const int c = (int)(i % (2 * D));
        if (c < D) k[r * D + c] = in[i];
        else v[r * D + c - D] = in[i];
    }
}

static int check_layout(const grl_kv_layout& kv) {
    GRL_REQUIRE(kv.k_pages && kv.v_pages && kv.block_table && kv.seq_lens, "NULL cache pointer");
    GRL_REQUIRE(kv.batch > 0 && kv.num_kv_heads > 0 && kv.page_tokens > 0 && kv.max_pages > 0, "bad cache shape");
    GRL_REQUIRE(kv.head_dim > 0 && kv.head_dim % 2 == 0 && kv.head_dim <= 256, "head_dim must be even and <= 256");
    GRL_REQUIRE(kv.cache_dtype == GRL_BF16 || kv.cache_dtype == GRL_F32 || kv.cache_dtype == GRL_FP8_INT4,
                "unknown cache dtype");
    if (kv.cache_dtype == GRL_FP8_INT4) {
        GRL_REQUIRE(kv.scales, "the quantised cache needs its scales buffer");
        GRL_REQUIRE(kv.head_dim % 32 == 0, "the quantised cache needs head_dim to be a multiple of 32 (scale groups)");
        GRL_REQUIRE(kv.page_tokens % 2 == 0, "the quantised cache stores value bytes by token pairs: page_tokens must be even");
    }
    return GRL_OK;
}

}  // namespace grl

using namespace grl;

extern "C" {

int grl_kv_append(grl_device* dev, const grl_append_params* p) {
    GRL_REQUIRE(dev && p, "NULL argument");
    int rc = check_layout(p->kv);
    if (rc) return rc;
    GRL_REQUIRE(p->k_new && p->v_new, "k_new / v_new is NULL");
    GRL_REQUIRE(p->n_new > 0, "n_new must be positive");
    GRL_REQUIRE(!p->q_in || (p->q_out && p->num_q_heads > 0), "q_in given without q_out / num_q_heads");
    GRL_REQUIRE(p->rope_mode >= GRL_ROPE_NONE && p->rope_mode <= GRL_ROPE_HALF, "unknown rope mode");
    DeviceGuard g(dev->ordinal);
    const grl_kv_layout& kv = p->kv;
    AppendArgs a{};
    a.k_pages = kv.k_pages; a.v_pages = kv.v_pages; a.block_table = kv.block_table; a.seq_lens = kv.seq_lens;
    a.k_new = p->k_new; a.v_new = p->v_new; a.q_in = p->q_in; a.q_out = p->q_out;
    a.B = kv.batch; a.Hkv = kv.num_kv_heads; a.Hq = p->num_q_heads; a.D = kv.head_dim; a.P = kv.page_tokens;
    a.max_pages = kv.max_pages; a.n_new = p->n_new;
    a.rope_mode = p->rope_mode; a.pos_base = p->pos_base; a.pos_offsets = p->pos_offsets;
    a.status = dev->d_status;
    a.scales = static_cast<uint16_t*>(kv.scales);
    dev->status_dirty = true;
    if (p->rope_mode != GRL_ROPE_NONE) a.freq = make_rope_freq(kv.head_dim, p->rope_theta, p->rope_scaling);
    if (kv.cache_dtype == GRL_FP8_INT4) {
        // K and V: one warp per (token, kv head, group of 32); the queries, if any, through the plain kernel
        const long long warps = (long long)p->n_new * kv.num_kv_heads * (kv.head_dim / 32);
        if (warps <= 32) {      // a decode step: one wide CTA per sequence does keys, values, queries and the length
            a.update_lens = p->update_lens ? 1 : 0;
            kv_append_quant_kernel<<<dim3(1, kv.batch), 1024, 0, dev->stream>>>(a);
            GRL_LAUNCHED("kv_append_quant_kernel");
            return GRL_OK;
        }
        int ctas = (int)((warps + 7) / 8);
        if (ctas > 1024) ctas = 1024;
        a.q_in = nullptr;       // bulk append: the queries go through the plain kernel below
        a.update_lens = 0;
        kv_append_quant_kernel<<<dim3(ctas, kv.batch), 256, 0, dev->stream>>>(a);
        GRL_LAUNCHED("kv_append_quant_kernel");
        a.q_in = p->q_in;
        if (p->q_in) {
            a.skip_kv = 1;
            a.update_lens = 0;
            const long long qitems = (long long)p->n_new * (kv.num_kv_heads + p->num_q_heads) * (kv.head_dim / 2);
            int qchunks = (int)((qitems + 4095) / 4096);
            if (qchunks > 128) qchunks = 128;
            kv_append_kernel<float><<<dim3(qchunks, kv.batch), 256, 0, dev->stream>>>(a);
            GRL_LAUNCHED("kv_append_kernel");
        }
        if (p->update_lens) {
            advance_lens_kernel<<<(kv.batch + 127) / 128, 128, 0, dev->stream>>>(kv.seq_lens, kv.batch, p->n_new,
                                                                                 kv.max_pages * kv.page_tokens);
            GRL_LAUNCHED("advance_lens_kernel");
        }
        return GRL_OK;
    }
    const long long items = (long long)p->n_new * (kv.num_kv_heads + (p->q_in ? p->num_q_heads : 0)) * (kv.head_dim / 2);
    // one CTA per sequence while a CTA has at most 16 items per thread (a decode step), more for bulk appends
    int chunks = (int)((items + 4095) / 4096);
    if (chunks > 128) chunks = 128;
    const bool fused_update = p->update_lens && chunks == 1;
    a.update_lens = fused_update ? 1 : 0;
    dim3 grid(chunks, kv.batch);
    // one chunk (the decode step): a wide CTA, so that every thread has only a few dependent load chains
    const int threads = chunks == 1 ? (items > 512 ? 1024 : 512) : 256;
    if (kv.cache_dtype == GRL_BF16) kv_append_kernel<__nv_bfloat16><<<grid, threads, 0, dev->stream>>>(a);
    else kv_append_kernel<float><<<grid, threads, 0, dev->stream>>>(a);
    GRL_LAUNCHED("kv_append_kernel");
    if (p->update_lens && !fused_update) {
        advance_lens_kernel<<<(kv.batch + 127) / 128, 128, 0, dev->stream>>>(kv.seq_lens, kv.batch, p->n_new,
                                                                                 kv.max_pages * kv.page_tokens);
        GRL_LAUNCHED("advance_lens_kernel");
    }
    return GRL_OK;
}

int grl_gemm_f32(grl_device* dev, const float* a, const float* b, float* c, int m, int k, int n) {
    GRL_REQUIRE(dev && a && b && c, "NULL argument");
    GRL_REQUIRE(m > 0 && k > 0 && n > 0, "bad shape (%d,%d,%d)", m, k, n);
    DeviceGuard g(dev->ordinal);
    gemm_f32_kernel<<<dim3((n + 15) / 16, (m + 15) / 16), 256, 0, dev->stream>>>(a, b, c, m, k, n);
    GRL_LAUNCHED("gemm_f32_kernel");
    return GRL_OK;
}

int grl_mla_concat(grl_device* dev, const float* k, const float* v, float* out, size_t rows, int head_dim) {
    GRL_REQUIRE(dev && k && v && out && rows > 0 && head_dim > 0, "bad argument");
    DeviceGuard g(dev->ordinal);
    const size_t blocks = (rows * 2 * head_dim + 255) / 256;
    mla_concat_kernel<<<(unsigned)(blocks < 4096 ? blocks : 4096), 256, 0, dev->stream>>>(k, v, out, rows, head_dim);
    GRL_LAUNCHED("mla_concat_kernel");
    return GRL_OK;
}

int grl_mla_split(grl_device* dev, const float* in, float* k, float* v, size_t rows, int head_dim) {
    GRL_REQUIRE(dev && k && v && in && rows > 0 && head_dim > 0, "bad argument");
    DeviceGuard g(dev->ordinal);
    const size_t blocks = (rows * 2 * head_dim + 255) / 256;
    mla_split_kernel<<<(unsigned)(blocks < 4096 ? blocks : 4096), 256, 0, dev->stream>>>(in, k, v, rows, head_dim);
    GRL_LAUNCHED("mla_split_kernel");
    return GRL_OK;
}

int grl_swizzle_kv(grl_device* dev, const float* in, float* out, int batch, int heads, int seq_len, int head_dim,
                   int wave, int reverse) {
    GRL_REQUIRE(dev && in && out, "NULL argument");
    GRL_REQUIRE(batch > 0 && heads > 0 && seq_len > 0 && head_dim > 0 && wave > 0, "bad shape");
    DeviceGuard g(dev->ordinal);
    const int s_pad = (seq_len + wave - 1) / wave * wave, d_pad = (head_dim + wave - 1) / wave * wave;
    const size_t total = (size_t)batch * heads * s_pad * d_pad;
    const size_t blocks = (total + 255) / 256;
    swizzle_kv_kernel<<<(unsigned)(blocks < 65535 * 16 ? blocks : 65535 * 16), 256, 0, dev->stream>>>(
        in, out, seq_len, head_dim, wave, s_pad, d_pad, total, reverse ? 1 : 0);
    GRL_LAUNCHED("swizzle_kv_kernel");
    return GRL_OK;
}

int grl_kv_gather(grl_device* dev, const grl_kv_layout* kv, int b, int n_tokens, float* out_k, float* out_v) {
    GRL_REQUIRE(dev && kv, "NULL argument");
    int rc = check_layout(*kv);
    if (rc) return rc;
    GRL_REQUIRE(b >= 0 && b < kv->batch, "sequence index out of range");
    GRL_REQUIRE(n_tokens >= 0 && n_tokens <= kv->max_pages * kv->page_tokens, "n_tokens out of range");
    if (n_tokens == 0) return GRL_OK;
    GRL_REQUIRE(out_k && out_v, "NULL output");
    DeviceGuard g(dev->ordinal);
    const size_t total = (size_t)n_tokens * kv->num_kv_heads * kv->head_dim;
    int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    if (kv->cache_dtype == GRL_FP8_INT4)
        kv_gather_quant_kernel<<<blocks, 256, 0, dev->stream>>>(
            (const uint8_t*)kv->k_pages, (const uint8_t*)kv->v_pages, (const uint16_t*)kv->scales, kv->block_table, b,
            n_tokens, kv->num_kv_heads, kv->head_dim, kv->page_tokens, kv->max_pages, out_k, out_v);
    else if (kv->cache_dtype == GRL_BF16)
        kv_gather_kernel<__nv_bfloat16><<<blocks, 256, 0, dev->stream>>>(
            (const __nv_bfloat16*)kv->k_pages, (const __nv_bfloat16*)kv->v_pages, kv->block_table, b, n_tokens,
            kv->num_kv_heads, kv->head_dim, kv->page_tokens, kv->max_pages, out_k, out_v);
    else
        kv_gather_kernel<float><<<blocks, 256, 0, dev->stream>>>(
            (const float*)kv->k_pages, (const float*)kv->v_pages, kv->block_table, b, n_tokens, kv->num_kv_heads,
            kv->head_dim, kv->page_tokens, kv->max_pages, out_k, out_v);
    GRL_LAUNCHED("kv_gather_kernel");
    return GRL_OK;
}

}  // extern "C"

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

static int check_layout(const grl_kv_layout& kv) {
    GRL_REQUIRE(kv.k_pages && kv.v_pages && kv.block_table && kv.seq_lens, "NULL cache pointer");
    GRL_REQUIRE(kv.batch > 0 && kv.num_kv_heads > 0 && kv.page_tokens > 0 && kv.max_pages > 0, "bad cache shape");
    GRL_REQUIRE(kv.head_dim > 0 && kv.head_dim % 2 == 0 && kv.head_dim <= 256, "head_dim must be even and <= 256");
    GRL_REQUIRE(kv.cache_dtype == GRL_BF16 || kv.cache_dtype == GRL_F32, "unknown cache dtype");
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
    dev->status_dirty = true;
    if (p->rope_mode != GRL_ROPE_NONE) a.freq = make_rope_freq(kv.head_dim, p->rope_theta, p->rope_scaling);
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
    if (kv->cache_dtype == GRL_BF16)
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

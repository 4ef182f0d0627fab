// GQA decode attention over the paged, head-major KV cache: split-KV partition over SMs plus a
// log-sum-exp merge.  Replaces shaders/gqa-attention.glsl:34-130 (scores -> softmax -> P.V in
// three global-memory phases with a (B,Hq,T) scratch) by a single streaming pass: every K and V
// row is read once with 16-byte loads and shared by all query heads of its KV group.
#include "common.cuh"

namespace grl {

bool decode_mma_supported(const grl_decode_params* p);
int decode_mma_launch(grl_device* dev, const grl_decode_params* p, int n_splits, float scale, bool direct, bool fuse);

constexpr float kEmptyMax = -1e30f;  // running max of a part that saw no token (finite on purpose)
constexpr int kDecodeThreads = 128;

struct DecodeArgs {
    const void* k_pages;
    const void* v_pages;
    const uint16_t* scales;   // quantised cache only: float16 bits per (row, group of 32)
    const int32_t* block_table;
    const int32_t* seq_lens;
    const float* q;
    float* part;       // [n_splits][rows*(D+2)]
    float* out;        // direct output when n_splits == 1 and no partial is wanted
    float* scores_out; // optional (B*Hq, scores_ld): scaled scores, natural-log domain
    int scores_ld;
    int B, Hq, Hkv, P, max_pages, n_splits, group, chunks;
    float scale;
    int direct;
};

template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float* x) {
        float4 v = __ldg(reinterpret_cast<const float4*>(p));
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float* x) {
        uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[2 * i] = __uint_as_float(w[i] << 16);
            x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// How a lane fetches its slice of one cached row (row = (page * Hkv + kv head) * page_tokens + slot) as float32.
template <typename T> struct KVLoad {
    static constexpr int VEC = Vec16<T>::N;
    __device__ static void load(const DecodeArgs& a, size_t row, int D, int li, float* kx, float* vx) {
        const size_t off = row * D + li * VEC;
        Vec16<T>::load(reinterpret_cast<const T*>(a.k_pages) + off, kx);
        Vec16<T>::load(reinterpret_cast<const T*>(a.v_pages) + off, vx);
    }
};
// GRL_FP8_INT4: 8 elements per lane = 8 key bytes, 4 value bytes and the scale of their group of 32; dequantised
// with the reference's arithmetic (cpp/src/ops/kv_cache.cpp:513-570): code value times 1/scale, the key scale
// for keys and values alike.
struct QuantKV {};
template <> struct KVLoad<QuantKV> {
    static constexpr int VEC = 8;
    __device__ static void load(const DecodeArgs& a, size_t row, int D, int li, float* kx, float* vx) {
        const uint2 kb = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(a.k_pages) + row * D + li * 8));
        // value bytes 4*li .. 4*li+3 of the token: two 16-bit halves of two words of its pair (quant_v_off)
        const int tok = (int)(row % (size_t)a.P);
        const uint8_t* vblock = reinterpret_cast<const uint8_t*>(a.v_pages) + (row - tok) * (size_t)(D / 2);
        const uint32_t vb = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(vblock + quant_v_off(tok, 4 * li, D))) |
                            ((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(vblock + quant_v_off(tok, 4 * li + 2, D))) << 16);
        const uint16_t hb = __ldg(a.scales + row * (D / 32) + (li >> 2));
        const uint32_t he = (hb >> 10) & 0x1Fu, hm = hb & 0x03FFu;
        const float scale = he == 0 ? (float)hm * 5.9604644775390625e-08f
                                    : __uint_as_float((((uint32_t)hb >> 15) << 31) | ((he + 112u) << 23) | (hm << 13));
        const float inv = scale > 0.f ? __fdiv_rn(1.0f, scale) : 1.0f;
        const uint32_t kw[2] = {kb.x, kb.y};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const uint32_t c = (kw[e >> 2] >> ((e & 3) * 8)) & 0xFFu;
            const uint32_t ce = (c >> 3) & 0x0Fu, cm = c & 7u;
            float v = ce == 0 ? (float)cm * 0.001953125f : __uint_as_float(((ce + 120u) << 23) | (cm << 20));
            v = (c & 0x80u) ? -v : v;
            kx[e] = __fmul_rn(v, inv);
            vx[e] = __fmul_rn((float)((int)((vb >> (e * 4)) & 0x0Fu) - 8), inv);
        }
    }
};

// grid (n_splits, Hkv*chunks, B); GC = query heads handled per CTA (a chunk of the KV group).
template <typename T, int D, int GC>
__global__ void __launch_bounds__(kDecodeThreads) decode_split_kernel(DecodeArgs a) {
    constexpr int VEC = KVLoad<T>::VEC;
    constexpr int LPT = D / VEC;           // lanes per token
    constexpr int TPW = 32 / LPT;          // tokens per warp iteration
    constexpr int NWARP = kDecodeThreads / 32;
    constexpr int NGRP = NWARP * TPW;      // independent online-softmax streams per CTA
    static_assert(LPT >= 1 && LPT <= 32, "head_dim / vector width");

    __shared__ float sm_m[NGRP][GC], sm_l[NGRP][GC];
    __shared__ float sm_acc[NGRP][GC][D];
    __shared__ float sm_w[NGRP][GC];

    const int split = blockIdx.x;
    const int kvh = blockIdx.y / a.chunks, chunk = blockIdx.y % a.chunks;
    const int b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane / LPT, li = lane % LPT;
    const int grp = warp * TPW + sub;
    const int qh0 = kvh * a.group + chunk * GC;          // first query head of this CTA
    const int n_heads = min(GC, a.group - chunk * GC);   // live heads in this chunk

    const int len = max(0, min(a.seq_lens[b], a.max_pages * a.P));   // never past the block table
    const int n_pages = (len + a.P - 1) / a.P;
    const int pps = (n_pages + a.n_splits - 1) / a.n_splits;  // pages per split
    const int t_begin = min(len, split * pps * a.P);
    const int t_end = min(len, (split + 1) * pps * a.P);

    float qv[GC][VEC], acc[GC][VEC], m[GC], l[GC];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
        m[g] = kEmptyMax;
        l[g] = 0.f;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            acc[g][e] = 0.f;
            qv[g][e] = (g < n_heads) ? a.q[((size_t)b * a.Hq + qh0 + g) * D + li * VEC + e] * a.scale : 0.f;
        }
    }

    const int32_t* bt = a.block_table + (size_t)b * a.max_pages;

    // The trip count is uniform across the warp (the shuffles below need all 32 lanes); a
    // lane group whose token index runs past the end just skips its update.
    for (int t0 = t_begin + warp * TPW; t0 < t_end; t0 += NGRP) {
        const int t = t0 + sub;
        const bool live = t < t_end;
        float kx[VEC], vx[VEC];
        if (live) {
            const int page = bt[t / a.P], slot = t % a.P;
            KVLoad<T>::load(a, ((size_t)page * a.Hkv + kvh) * a.P + slot, D, li, kx, vx);
        } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) { kx[e] = 0.f; vx[e] = 0.f; }
        }
        float s[GC];
#pragma unroll
        for (int g = 0; g < GC; ++g) {
            float d = 0.f;
#pragma unroll
            for (int e = 0; e < VEC; ++e) d = fmaf(qv[g][e], kx[e], d);
            s[g] = d;
        }
#pragma unroll
        for (int off2 = 1; off2 < LPT; off2 <<= 1)
#pragma unroll
            for (int g = 0; g < GC; ++g) s[g] += __shfl_xor_sync(0xffffffffu, s[g], off2);
        if (live && a.scores_out && li == 0) {
#pragma unroll
            for (int g = 0; g < GC; ++g)
                if (g < n_heads) a.scores_out[((size_t)b * a.Hq + qh0 + g) * a.scores_ld + t] = s[g];
        }
        if (live) {
#pragma unroll
            for (int g = 0; g < GC; ++g) {
                const float m_new = fmaxf(m[g], s[g]);
                const float corr = __expf(m[g] - m_new);
                const float p = __expf(s[g] - m_new);
                l[g] = l[g] * corr + p;
                m[g] = m_new;
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[g][e] = fmaf(acc[g][e], corr, p * vx[e]);
            }
        }
    }

    // combine the NGRP streams of this CTA
#pragma unroll
    for (int g = 0; g < GC; ++g) {
        if (li == 0) { sm_m[grp][g] = m[g]; sm_l[grp][g] = l[g]; }
#pragma unroll
        for (int e = 0; e < VEC; ++e) sm_acc[grp][g][li * VEC + e] = acc[g][e];
    }
    __syncthreads();
    __shared__ float sm_mtot[GC], sm_ltot[GC];
    if (tid < GC) {
        float mt = kEmptyMax;
        for (int i = 0; i < NGRP; ++i) mt = fmaxf(mt, sm_m[i][tid]);
        float lt = 0.f;
        for (int i = 0; i < NGRP; ++i) {
            float w = __expf(sm_m[i][tid] - mt);
            sm_w[i][tid] = w;
            lt += w * sm_l[i][tid];
        }
        sm_mtot[tid] = mt;
        sm_ltot[tid] = lt;
    }
    __syncthreads();
    const int rows = a.B * a.Hq;
    for (int idx = tid; idx < n_heads * D; idx += kDecodeThreads) {
        const int g = idx / D, d = idx % D;
        float o = 0.f;
#pragma unroll 4
        for (int i = 0; i < NGRP; ++i) o = fmaf(sm_w[i][g], sm_acc[i][g][d], o);
        const int row = b * a.Hq + qh0 + g;
        if (a.direct) {
            const float lt = sm_ltot[g];
            a.out[(size_t)row * D + d] = lt > 0.f ? o / lt : 0.f;
        } else {
            float* part = a.part + (size_t)split * rows * (D + 2);
            part[(size_t)row * D + d] = o;
            if (d == 0) {
                part[(size_t)rows * D + row] = sm_mtot[g];
                part[(size_t)rows * D + rows + row] = sm_ltot[g];
            }
        }
    }
}

// parts: n_parts x [O (rows*D) | m (rows) | l (rows)].  grid (rows), block 128.
// Stage 1: the block finds the common maximum and the weights e^{m_i - m} of up to 1024 parts
// (kept in shared memory); stage 2: each thread owns output columns and sums the parts with four
// independent accumulators, so that the loads of different parts are in flight together.
constexpr int kMaxMergeParts = 1024;
__global__ void __launch_bounds__(128) lse_merge_kernel(const float* __restrict__ parts, int n_parts,
                                                         size_t part_stride, int rows, int D, int normalise,
                                                         float* __restrict__ out) {
    __shared__ float sm_w[kMaxMergeParts];
    __shared__ float sm_red[4];
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* ml = parts + (size_t)rows * D;
    float mloc = kEmptyMax;
    for (int i = tid; i < n_parts; i += 128) {
        const float m = ml[i * part_stride + row];
        sm_w[i] = m;
        mloc = fmaxf(mloc, m);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, off));
    if (lane == 0) sm_red[warp] = mloc;
    __syncthreads();
    const float mt = fmaxf(fmaxf(sm_red[0], sm_red[1]), fmaxf(sm_red[2], sm_red[3]));
    __syncthreads();
    float lloc = 0.f;
    for (int i = tid; i < n_parts; i += 128) {
        const float w = __expf(sm_w[i] - mt);
        sm_w[i] = w;
        lloc = fmaf(w, ml[i * part_stride + rows + row], lloc);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) lloc += __shfl_xor_sync(0xffffffffu, lloc, off);
    if (lane == 0) sm_red[warp] = lloc;
    __syncthreads();
    const float lt = (sm_red[0] + sm_red[1]) + (sm_red[2] + sm_red[3]);
    for (int d = tid; d < D; d += 128) {
        const float* p = parts + (size_t)row * D + d;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        int i = 0;
        for (; i + 4 <= n_parts; i += 4) {
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = fmaf(sm_w[i + e], p[(size_t)(i + e) * part_stride], acc[e]);
        }
        for (; i < n_parts; ++i) acc[0] = fmaf(sm_w[i], p[(size_t)i * part_stride], acc[0]);
        const float o = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        if (normalise) out[(size_t)row * D + d] = lt > 0.f ? o / lt : 0.f;
        else out[(size_t)row * D + d] = o;
    }
    if (!normalise && tid == 0) {
        out[(size_t)rows * D + row] = mt;
        out[(size_t)rows * D + rows + row] = lt;
    }
}

template <typename T, int D, int GC>
static int launch_decode(grl_device* dev, const DecodeArgs& a) {
    dim3 grid(a.n_splits, a.Hkv * a.chunks, a.B);
    decode_split_kernel<T, D, GC><<<grid, kDecodeThreads, 0, dev->stream>>>(a);
    GRL_LAUNCHED("decode_split_kernel");
    return GRL_OK;
}

template <typename T, int D>
static int dispatch_gc(grl_device* dev, DecodeArgs& a) {
    int gc = a.group <= 1 ? 1 : a.group <= 2 ? 2 : a.group <= 4 ? 4 : 8;
    a.chunks = (a.group + gc - 1) / gc;
    switch (gc) {
        case 1: return launch_decode<T, D, 1>(dev, a);
        case 2: return launch_decode<T, D, 2>(dev, a);
        case 4: return launch_decode<T, D, 4>(dev, a);
        default: return launch_decode<T, D, 8>(dev, a);
    }
}

template <typename T>
static int dispatch_decode_d(grl_device* dev, DecodeArgs& a, int D) {
    switch (D) {
        case 32: return dispatch_gc<T, 32>(dev, a);
        case 64: return dispatch_gc<T, 64>(dev, a);
        case 128: return dispatch_gc<T, 128>(dev, a);
        default: return set_error(GRL_ERR_UNSUPPORTED, "head_dim %d not supported (32, 64 or 128)", D);
    }
}

static int check_decode(const grl_decode_params* p, bool need_tensors = true) {
    GRL_REQUIRE(p, "params is NULL");
    const grl_kv_layout& kv = p->kv;
    GRL_REQUIRE(kv.k_pages && kv.v_pages && kv.block_table && kv.seq_lens, "NULL cache pointer");
    GRL_REQUIRE(kv.batch > 0 && kv.num_kv_heads > 0 && kv.page_tokens > 0 && kv.max_pages > 0, "bad cache shape");
    GRL_REQUIRE(p->num_q_heads > 0 && p->num_q_heads % kv.num_kv_heads == 0,
                "num_q_heads (%d) must be a multiple of num_kv_heads (%d)", p->num_q_heads, kv.num_kv_heads);
    GRL_REQUIRE(kv.cache_dtype == GRL_BF16 || kv.cache_dtype == GRL_F32 || kv.cache_dtype == GRL_FP8_INT4,
                "unknown cache dtype");
    GRL_REQUIRE(kv.cache_dtype != GRL_FP8_INT4 || (kv.scales && kv.head_dim % 32 == 0),
                "the quantised cache needs its scales buffer and a head_dim that is a multiple of 32");
    if (need_tensors) {
        GRL_REQUIRE(p->q, "q is NULL");
        GRL_REQUIRE(p->out || p->partial_out, "out and partial_out are both NULL");
        const int bound = p->max_seq_len > 0 ? p->max_seq_len : kv.max_pages * kv.page_tokens;
        GRL_REQUIRE(!p->scores_out || p->scores_ld >= bound, "scores_ld %d is below the sequence bound %d",
                    p->scores_ld, bound);
    }
    return GRL_OK;
}

}  // namespace grl

using namespace grl;

extern "C" {

int grl_decode_pick_splits(grl_device* dev, const grl_decode_params* p, int* n_splits) {
    GRL_REQUIRE(dev && n_splits, "NULL argument");
    int rc = check_decode(p, false);
    if (rc) return rc;
    if (p->n_splits > 0) {
        *n_splits = p->n_splits;
        return GRL_OK;
    }
    const grl_kv_layout& kv = p->kv;
    const int max_len = p->max_seq_len > 0 ? p->max_seq_len : kv.max_pages * kv.page_tokens;
    const bool generic = !decode_mma_supported(p) || p->force_simt;
    // the tensor-core kernel walks 64-token stages whatever the page size
    const int unit = generic ? kv.page_tokens : 64;
    const int pages = (max_len + unit - 1) / unit;
    const int base_ctas = kv.batch * kv.num_kv_heads;
    // At most one CTA per SM: that already keeps HBM saturated (three 32 KB stages in flight each), and one
    // CTA more than there are SMs makes a pair share an SM and finish last.  Measured on B200, B1 x 8 KV
    // heads x 131072 tokens: 87 us with 18 splits (144 CTAs), 94 us with 19 (152), 100 us with 64; B32 x 8
    // heads x 4096 tokens is fastest unsplit.
    const int sms = dev->prop.multiProcessorCount;
    // The generic kernel (128-thread CTAs, no shared-memory ring) wants several CTAs per SM to hide its loads and,
    // over a quantised cache, its dequantising arithmetic: aim at eight per SM.
    int s = generic ? (8 * sms + base_ctas - 1) / base_ctas : sms / base_ctas;
    if (s > pages / 2) s = pages / 2;          // every split keeps at least 2 pages
    if (s > 256) s = 256;
    if (s < 1) s = 1;
    *n_splits = s;
    return GRL_OK;
}

int grl_decode_workspace_bytes(const grl_decode_params* p, int n_splits, size_t* bytes) {
    GRL_REQUIRE(p && bytes && n_splits > 0, "bad argument");
    const size_t rows = (size_t)p->kv.batch * p->num_q_heads;
    *bytes = sizeof(float) * (size_t)n_splits * rows * (p->kv.head_dim + 2);
    return GRL_OK;
}

int grl_lse_merge(grl_device* dev, const float* parts, int n_parts, size_t part_stride, int rows,
                  int head_dim, int normalise, float* out) {
    GRL_REQUIRE(dev && parts && out, "NULL argument");
    GRL_REQUIRE(n_parts > 0 && rows > 0 && head_dim > 0, "bad shape");
    GRL_REQUIRE(n_parts <= kMaxMergeParts, "at most %d parts can be merged in one call", kMaxMergeParts);
    GRL_REQUIRE(part_stride >= (size_t)rows * (head_dim + 2), "part_stride too small");
    DeviceGuard g(dev->ordinal);
    lse_merge_kernel<<<rows, 128, 0, dev->stream>>>(parts, n_parts, part_stride, rows, head_dim, normalise, out);
    GRL_LAUNCHED("lse_merge_kernel");
    return GRL_OK;
}

int grl_gqa_decode(grl_device* dev, const grl_decode_params* p) {
    GRL_REQUIRE(dev, "dev is NULL");
    int rc = check_decode(p);
    if (rc) return rc;
    int n_splits = 0;
    rc = grl_decode_pick_splits(dev, p, &n_splits);
    if (rc) return rc;
    const grl_kv_layout& kv = p->kv;
    const int D = kv.head_dim;
    const bool direct = (n_splits == 1) && !p->partial_out && !p->exchange;
    size_t need = 0;
    grl_decode_workspace_bytes(p, n_splits, &need);
    if (!direct)
        GRL_REQUIRE(p->workspace && p->workspace_bytes >= need, "decode workspace too small: %zu < %zu",
                    p->workspace_bytes, need);
    DeviceGuard g(dev->ordinal);
    DecodeArgs a{};
    a.k_pages = kv.k_pages; a.v_pages = kv.v_pages; a.scales = static_cast<const uint16_t*>(kv.scales); a.block_table = kv.block_table; a.seq_lens = kv.seq_lens;
    a.q = p->q; a.part = (float*)p->workspace; a.out = p->out;
    a.scores_out = p->scores_out; a.scores_ld = p->scores_ld;
    a.B = kv.batch; a.Hq = p->num_q_heads; a.Hkv = kv.num_kv_heads; a.P = kv.page_tokens;
    a.max_pages = kv.max_pages; a.n_splits = n_splits; a.group = p->num_q_heads / kv.num_kv_heads;
    a.scale = p->scale == 0.f ? 1.f / sqrtf((float)D) : p->scale;
    a.direct = direct ? 1 : 0;
    const bool mma = decode_mma_supported(p) && !p->force_simt;
    // the tensor-core kernel merges its own splits (last CTA of a head to arrive) when its counters can hold the heads
    const bool fused = mma && !direct && n_splits <= 256 && kv.batch * kv.num_kv_heads <= grl_device::kCounterSlots;
    GRL_REQUIRE(!p->exchange || fused,
                "the cross-GPU merge inside the decode needs the tensor-core geometry (bf16 cache at head_dim 128 / 64 or "
                "the quantised cache at 128, pages of 64 / 32 / 16 tokens, at most 8 query heads per kv head) and a split "
                "launch; use partial_out and grl_exchange_merge instead");
    if (mma)
        rc = decode_mma_launch(dev, p, n_splits, a.scale, direct, fused);
    else
        rc = kv.cache_dtype == GRL_BF16       ? dispatch_decode_d<__nv_bfloat16>(dev, a, D)
             : kv.cache_dtype == GRL_FP8_INT4 ? dispatch_decode_d<QuantKV>(dev, a, D)
                                              : dispatch_decode_d<float>(dev, a, D);
    if (rc || direct || fused) return rc;
    const int rows = kv.batch * p->num_q_heads;
    const size_t stride = (size_t)rows * (D + 2);
    if (p->partial_out)
        return grl_lse_merge(dev, (const float*)p->workspace, n_splits, stride, rows, D, 0, p->partial_out);
    return grl_lse_merge(dev, (const float*)p->workspace, n_splits, stride, rows, D, 1, p->out);
}

// ---------------------------------------------------------------------------------------------
// Decode without any allocation by anyone.
//
// Some hosts of this library cannot give the decode step a workspace: a serving process that
// hands every byte of device memory to its own arena at start-up and treats a later cudaMalloc
// as a bug (it synchronises the device and can fail when the arena already owns the memory), or
// a plugin loaded into such a process that is only ever given its input and output tensors.
// For them the split-KV partials live in the array below, which is part of the library's image:
// every GPU that loads the library holds these 4 MiB until the process exits.
constexpr size_t kStaticScratchFloats = 1u << 20;   // 4 MiB
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];
static float* g_decode_scratch_addr[64];            // per device ordinal: device address of the array
static std::mutex g_decode_scratch_mu;

int grl_gqa_decode_static(grl_device* dev, const grl_decode_params* p) {
    GRL_REQUIRE(dev && p, "NULL argument");
    GRL_REQUIRE(dev->ordinal >= 0 && dev->ordinal < 64, "device ordinal %d out of range", dev->ordinal);
    int n_splits = 0;
    int rc = grl_decode_pick_splits(dev, p, &n_splits);
    if (rc) return rc;
    size_t need = 0;
    rc = grl_decode_workspace_bytes(p, n_splits, &need);
    if (rc) return rc;
    // an unsplit launch writes its result directly and touches no scratch, whatever its nominal size
    const bool unsplit = (n_splits == 1) && !p->partial_out && !p->exchange;
    if (!unsplit && need > kStaticScratchFloats * sizeof(float))
        return set_error(GRL_ERR_INVALID,
                         "grl_gqa_decode_static: %d splits x %d rows need %zu bytes of scratch, the built-in array holds "
                         "%zu; pass fewer splits (n_splits) or use grl_gqa_decode with a caller workspace",
                         n_splits, p->kv.batch * p->num_q_heads, need, kStaticScratchFloats * sizeof(float));
    float* scratch = nullptr;
    {
        // In host code the array's name is only a stand-in; the kernels need its device address on
        // THIS device, asked for once per device with that device current.
        std::lock_guard<std::mutex> lock(g_decode_scratch_mu);
        scratch = g_decode_scratch_addr[dev->ordinal];
        if (!scratch) {
            DeviceGuard g(dev->ordinal);
            GRL_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_decode_scratch));
            g_decode_scratch_addr[dev->ordinal] = scratch;
        }
    }
    grl_decode_params q = *p;
    q.n_splits = n_splits;
    q.workspace = scratch;
    q.workspace_bytes = kStaticScratchFloats * sizeof(float);
    return grl_gqa_decode(dev, &q);
}

}  // extern "C"

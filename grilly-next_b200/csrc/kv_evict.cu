// Eviction on the paged KV cache: H2O selection, the heuristic branch of speculative eviction, and
// compaction.  Replaces the host loops of kvCacheEvictH2O (cpp/src/ops/kv_cache.cpp:595-634),
// kvCacheEvictSpeculative's fallback (:905-929) and kvCacheCompact (:941-992), which in the reference
// walk persistently mapped metadata on the CPU; here the metadata (cumulative score, tombstone) and the
// K/V rows live in HBM and every step is a kernel.  Everything is exact: the column sums add in the
// reference's order (one thread per cached token walks the query rows), selection is a radix select on
// the float bit patterns with ties going to the lowest index, and rows move as raw bytes.
#include "common.cuh"

namespace grl {
namespace evict {

constexpr int kThreads = 1024;

// float -> uint32 whose unsigned order is the float order
__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// cum[b][t] += sum_q attn[b][q][t], the sum over q taken in ascending q with plain float adds
// (kv_cache.cpp:606-615).
__global__ void score_accumulate_kernel(const float* __restrict__ attn, int q_rows, int ld, const int32_t* seq_lens,
                                        float* cum, int capacity) {
    const int b = blockIdx.y;
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    const int len = max(0, min(seq_lens[b], capacity));   // never past the metadata arrays
    if (t >= len || t >= ld) return;
    const float* col = attn + (size_t)b * q_rows * ld + t;
    float acc = 0.f;
    for (int q = 0; q < q_rows; ++q) acc = __fadd_rn(acc, col[(size_t)q * ld]);
    float* c = cum + (size_t)b * capacity + t;
    *c = __fadd_rn(*c, acc);
}

// cum[b][t] += sum_h exp(scores[b][h][t] - m[b][h]) / l[b][h]: the attention mass token t received from
// the Hq query heads of one decode step.  (m, l) come from the step's un-normalised partial [O | m | l].
__global__ void mass_accumulate_kernel(const float* __restrict__ scores, int ld, const float* __restrict__ partial,
                                       int Hq, int D, int rows, const int32_t* seq_lens, float* cum, int capacity) {
    extern __shared__ float s_ml[];          // [Hq] m, [Hq] 1/l
    const int b = blockIdx.y;
    const int len = max(0, min(seq_lens[b], capacity));   // never past the metadata arrays
    for (int h = threadIdx.x; h < Hq; h += blockDim.x) {
        const int row = b * Hq + h;
        const float l = partial[(size_t)rows * D + rows + row];
        s_ml[h] = partial[(size_t)rows * D + row];
        s_ml[Hq + h] = l > 0.f ? 1.f / l : 0.f;
    }
    __syncthreads();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= len) return;
    float acc = 0.f;
    for (int h = 0; h < Hq; ++h)
        acc += __expf(scores[((size_t)b * Hq + h) * ld + t] - s_ml[h]) * s_ml[Hq + h];
    cum[(size_t)b * capacity + t] += acc;
}

// block-wide exclusive scan of one int per thread; returns the exclusive prefix, *total = block sum
__device__ __forceinline__ int block_exclusive_scan(int v, int* total, int* s_warp /* [33] */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += n;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = lane < (int)(blockDim.x >> 5) ? s_warp[lane] : 0;
        int winc = w;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, winc, d);
            if (lane >= d) winc += n;
        }
        s_warp[lane] = winc - w;                 // exclusive prefix of the warp sums
        if (lane == 31) s_warp[32] = winc;       // block total
    }
    __syncthreads();
    const int ex = s_warp[warp] + inc - v;
    *total = s_warp[32];
    __syncthreads();                             // s_warp is reused by the next call
    return ex;
}

// One CTA per sequence: tombstone the num_evict tokens of [0, len) with the lowest cumulative score,
// ties to the lowest index (kv_cache.cpp:618-633; std::partial_sort leaves the order of ties open).
__global__ void __launch_bounds__(kThreads) evict_lowest_kernel(const float* __restrict__ cum, uint8_t* tomb,
                                                               const int32_t* seq_lens, int capacity, int num_evict) {
    __shared__ int s_hist[256];
    __shared__ int s_warp[33];
    __shared__ uint32_t s_prefix;
    __shared__ int s_k;
    const int b = blockIdx.x, tid = threadIdx.x;
    const int len = max(0, min(seq_lens[b], capacity));   // never past the metadata arrays
    int k = num_evict > 0 ? num_evict : len / 4;          // default: a quarter (kv_cache.cpp:598-600)
    if (k <= 0 || k >= len) return;                       // kv_cache.cpp:601
    const float* c = cum + (size_t)b * capacity;
    uint8_t* tb = tomb + (size_t)b * capacity;
    // radix select, most significant byte first: after the four passes `prefix` is the key of the k-th
    // smallest element and k has become its rank among the elements equal to it
    if (tid == 0) { s_prefix = 0; s_k = k; }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int i = tid; i < 256; i += kThreads) s_hist[i] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int t = tid; t < len; t += kThreads) {
            const uint32_t key = order_key(c[t]);
            if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int kk = s_k, bin = 0;
            for (; bin < 256; ++bin) {
                if (kk <= s_hist[bin]) break;
                kk -= s_hist[bin];
            }
            s_prefix = prefix | ((uint32_t)bin << shift);
            s_k = kk;
        }
        __syncthreads();
    }
    const uint32_t kth = s_prefix;
    const int need_equal = s_k;        // how many of the elements equal to kth go, in index order
    int taken = 0;                     // equal elements tombstoned so far (same in every thread)
    for (int base = 0; base < len; base += kThreads) {
        const int t = base + tid;
        const uint32_t key = t < len ? order_key(c[t]) : 0xffffffffu;
        const int eq = (t < len && key == kth) ? 1 : 0;
        int total;
        const int rank = block_exclusive_scan(eq, &total, s_warp);
        if (t < len && (key < kth || (eq && taken + rank < need_equal))) tb[t] = 1;
        taken += total;
    }
}

// Heuristic of kvCacheEvictSpeculative without a trained head (kv_cache.cpp:905-929): relevance =
// 0.7 * cum / max(cum) + 0.3 * t / len; tombstone below the threshold.  The maximum runs over every
// token of [0, len), tombstoned or not, and starts from 0 as the reference's does.
__global__ void __launch_bounds__(kThreads) evict_heuristic_kernel(const float* __restrict__ cum, uint8_t* tomb,
                                                                  float* relevance, const int32_t* seq_lens,
                                                                  int capacity, float threshold) {
    __shared__ float s_max[32];
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int len = max(0, min(seq_lens[b], capacity));   // never past the metadata arrays
    const float* c = cum + (size_t)b * capacity;
    float m = 0.f;
    for (int t = tid; t < len; t += kThreads) m = fmaxf(m, c[t]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    if (lane == 0) s_max[warp] = m;
    __syncthreads();
    m = s_max[0];
    for (int w = 1; w < kThreads / 32; ++w) m = fmaxf(m, s_max[w]);
    const float inv = m > 0.f ? __fdiv_rn(1.f, m) : 1.f;
    for (int t = tid; t < len; t += kThreads) {
        if (tomb[(size_t)b * capacity + t]) continue;
        const float norm = __fmul_rn(c[t], inv);
        const float rec = __fdiv_rn((float)t, (float)len);
        const float rel = __fadd_rn(__fmul_rn(0.7f, norm), __fmul_rn(0.3f, rec));
        if (relevance) relevance[(size_t)b * capacity + t] = rel;
        if (rel < threshold) tomb[(size_t)b * capacity + t] = 1;
    }
}

// One CTA per sequence: new_pos[t] = number of live tokens before t (or -1 for a tombstone), live count
// to new_len[b].
__global__ void __launch_bounds__(kThreads) compact_scan_kernel(const uint8_t* __restrict__ tomb,
                                                               const int32_t* seq_lens, int capacity,
                                                               int32_t* new_pos, int32_t* new_len) {
    __shared__ int s_warp[33];
    const int b = blockIdx.x, tid = threadIdx.x;
    const int len = max(0, min(seq_lens[b], capacity));   // never past the metadata arrays
    int carried = 0;
    for (int base = 0; base < len; base += kThreads) {
        const int t = base + tid;
        const int live = (t < len && !tomb[(size_t)b * capacity + t]) ? 1 : 0;
        int total;
        const int ex = block_exclusive_scan(live, &total, s_warp);
        if (t < len) new_pos[(size_t)b * capacity + t] = live ? carried + ex : -1;
        carried += total;
    }
    if (tid == 0) new_len[b] = carried;
}

struct MoveArgs {
    uint8_t* k_pages;
    uint8_t* v_pages;
    const int32_t* block_table;
    const int32_t* seq_lens;     // lengths BEFORE compaction
    const int32_t* new_pos;
    int Hkv, P, max_pages, capacity, row_bytes;
};

// One CTA per (kv head, sequence, K|V, column part) walks the sequence in tiles of 2048 16-byte vectors:
// load the live rows of the tile, ONE barrier, store them at their new positions.  new_pos[t] <= t and order
// is kept, so the rows a tile writes lie at or before the rows it read and strictly before anything a later
// tile reads -- the in-order loop of kv_cache.cpp:957-989, one head at a time; the barrier only has to
// separate a tile's loads from its own stores.  Column ranges of a row are independent of one another, so
// wide rows are cut in two for twice the CTAs (the walk itself is sequential).  The block table sits in
// shared memory and the next tile's new positions are fetched before the barrier, so that a tile costs one
// dependent global load (the row itself), not three.
constexpr int kMoveThreads = 256, kMovePerThread = 8, kMoveBtSmem = 2048;
__global__ void __launch_bounds__(kMoveThreads, 3) compact_move_kernel(MoveArgs a) {
    __shared__ int32_t s_bt[kMoveBtSmem];
    const int h = blockIdx.x, b = blockIdx.y;
    const int parts = gridDim.z / 2, part = blockIdx.z >> 1;
    uint8_t* pool = (blockIdx.z & 1) == 0 ? a.k_pages : a.v_pages;
    const int len = max(0, min(a.seq_lens[b], min(a.capacity, a.max_pages * a.P)));   // never past the block table
    const int32_t* bt_g = a.block_table + (size_t)b * a.max_pages;
    const int32_t* np = a.new_pos + (size_t)b * a.capacity;
    const int n_pages = (len + a.P - 1) / a.P;
    const bool bt_in_smem = n_pages <= kMoveBtSmem;
    if (bt_in_smem)
        for (int i = threadIdx.x; i < n_pages; i += kMoveThreads) s_bt[i] = bt_g[i];
    __syncthreads();
    const int32_t* bt = bt_in_smem ? s_bt : bt_g;
    const int vpr = a.row_bytes / 16 / parts;                  // 16-byte vectors of a row that this CTA moves
    const int v0 = part * vpr;
    const int tile_rows = kMoveThreads * kMovePerThread / vpr;
    auto vec_ptr = [&](int t, int v) -> uint4* {
        const size_t page = (size_t)bt[t / a.P];
        return reinterpret_cast<uint4*>(pool + ((page * a.Hkv + h) * a.P + (t % a.P)) * (size_t)a.row_bytes) + v0 + v;
    };
    uint4 regs[kMovePerThread];
    int dst[kMovePerThread], nxt[kMovePerThread];
#pragma unroll
    for (int i = 0; i < kMovePerThread; ++i) {                 // new positions of the first tile
        const int t = (threadIdx.x + i * kMoveThreads) / vpr;
        nxt[i] = t < len ? np[t] : -1;
    }
    for (int base = 0; base < len; base += tile_rows) {
#pragma unroll
        for (int i = 0; i < kMovePerThread; ++i) {
            const int idx = threadIdx.x + i * kMoveThreads;
            const int t = base + idx / vpr;
            dst[i] = (t < len && nxt[i] != t) ? nxt[i] : -1;   // -1: tombstone, past the end, or already in place
            if (dst[i] >= 0) regs[i] = *vec_ptr(t, idx % vpr);
        }
#pragma unroll
        for (int i = 0; i < kMovePerThread; ++i) {             // the next tile's positions travel with this tile's rows
            const int t = base + tile_rows + (threadIdx.x + i * kMoveThreads) / vpr;
            nxt[i] = t < len ? np[t] : -1;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kMovePerThread; ++i)
            if (dst[i] >= 0) *vec_ptr(dst[i], (threadIdx.x + i * kMoveThreads) % vpr) = regs[i];
    }
}

// One CTA per sequence, after the rows have moved: compact the scores the same way, clear the
// tombstones, zero the scores of the freed tail, publish the new length and the evicted count.
__global__ void __launch_bounds__(kThreads) compact_meta_kernel(float* cum, uint8_t* tomb, float* relevance,
                                                               int32_t* seq_lens, int32_t* evicted,
                                                               const int32_t* new_pos, const int32_t* new_len,
                                                               int capacity) {
    const int b = blockIdx.x, tid = threadIdx.x;
    const int len = max(0, min(seq_lens[b], capacity)), nl = new_len[b];
    float* c = cum + (size_t)b * capacity;
    float* r = relevance ? relevance + (size_t)b * capacity : nullptr;
    const int32_t* np = new_pos + (size_t)b * capacity;
    for (int base = 0; base < len; base += kThreads) {
        const int t = base + tid;
        const bool mv = t < len && np[t] >= 0;
        const float v = mv ? c[t] : 0.f;
        const float rv = (mv && r) ? r[t] : 0.f;
        __syncthreads();
        if (mv) { c[np[t]] = v; if (r) r[np[t]] = rv; }
        __syncthreads();
    }
    for (int t = tid; t < len; t += kThreads) {
        tomb[(size_t)b * capacity + t] = 0;
        if (t >= nl) { c[t] = 0.f; if (r) r[t] = 0.f; }
    }
    __syncthreads();
    if (tid == 0) {
        seq_lens[b] = nl;
        if (evicted) evicted[b] += len - nl;
    }
}

// ---------------------------------------------------------------------------------------------
// Trainable eviction head (kv_cache.cpp:636-845,856-903): relevance = sigmoid(W2 . relu(W1^T x + b1) + b2)
// for one sequence.  The reference runs it token by token on the CPU; here a token is a thread in the
// forward pass and a parameter is a thread in the gradient pass, each walking its sum in the
// reference's order with unfused multiplies and adds, so only exp() separates the two.

// received[t] = sum_q attn[q][t] (ascending q), one thread per token
__global__ void head_received_kernel(const float* __restrict__ attn, int seq_len, int T, float* received) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    float acc = 0.f;
    for (int q = 0; q < seq_len; ++q) acc = __fadd_rn(acc, attn[(size_t)q * T + t]);
    received[t] = acc;
}

// One CTA: median[0] = the element std::nth_element would leave at index T/2 (the (T/2+1)-th smallest)
__global__ void __launch_bounds__(kThreads) head_median_kernel(const float* __restrict__ received, int T, float* median) {
    __shared__ int s_hist[256];
    __shared__ uint32_t s_prefix;
    __shared__ int s_k;
    const int tid = threadIdx.x;
    if (tid == 0) { s_prefix = 0; s_k = T / 2 + 1; }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int i = tid; i < 256; i += kThreads) s_hist[i] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int t = tid; t < T; t += kThreads) {
            const uint32_t key = order_key(received[t]);
            if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int kk = s_k, bin = 0;
            for (; bin < 256; ++bin) {
                if (kk <= s_hist[bin]) break;
                kk -= s_hist[bin];
            }
            s_prefix = prefix | ((uint32_t)bin << shift);
            s_k = kk;
        }
        __syncthreads();
    }
    if (tid == 0) {
        const uint32_t key = s_prefix;
        const uint32_t u = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
        median[0] = __uint_as_float(u);
    }
}

struct HeadArgs {
    const float* w1; const float* b1; const float* w2; const float* b2;
    int in_dim, h_dim;
};

// Forward pass, one thread per live token: hidden (kept for the gradient pass), score -> relevance,
// dlogit = score - label (train) or tombstone below the threshold (predict).
__global__ void head_forward_kernel(HeadArgs hd, const float* __restrict__ feat, int T, const uint8_t* tomb_in,
                                    float* relevance, float* hidden, float* dlogit, const float* received,
                                    const float* median, uint8_t* tomb_out, float threshold) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    if (tomb_in[t]) {                       // skipped by the reference: contributes nothing
        if (dlogit) dlogit[t] = 0.f;
        if (hidden) for (int h = 0; h < hd.h_dim; ++h) hidden[(size_t)t * hd.h_dim + h] = 0.f;
        return;
    }
    const float* x = feat + (size_t)t * hd.in_dim;
    float logit = hd.b2[0];
    for (int h = 0; h < hd.h_dim; ++h) {
        float sum = hd.b1[h];
        for (int i = 0; i < hd.in_dim; ++i) sum = __fadd_rn(sum, __fmul_rn(hd.w1[(size_t)i * hd.h_dim + h], x[i]));
        const float hv = fmaxf(0.f, sum);
        if (hidden) hidden[(size_t)t * hd.h_dim + h] = hv;
        logit = __fadd_rn(logit, __fmul_rn(hd.w2[h], hv));
    }
    const float score = __fdiv_rn(1.f, __fadd_rn(1.f, expf(-logit)));
    relevance[t] = score;
    if (dlogit) dlogit[t] = __fadd_rn(score, received[t] > median[0] ? -1.f : -0.f);
    if (tomb_out && score < threshold) tomb_out[t] = 1;
}

// Gradient pass + SGD step, one thread per parameter, tokens in ascending order:
// index < in*h: W1[i][h]; then b1[h]; then W2[h]; then b2.
__global__ void head_update_kernel(float* w1, float* b1, float* w2, float* b2, int in_dim, int h_dim,
                                   const float* __restrict__ feat, const float* __restrict__ hidden,
                                   const float* __restrict__ dlogit, const float* __restrict__ w2_old, int T, float step) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int n_w1 = in_dim * h_dim;
    if (idx >= n_w1 + 2 * h_dim + 1) return;
    float g = 0.f;
    if (idx < n_w1 + h_dim) {               // W1[i][h] or b1[h]: through the ReLU
        const bool bias = idx >= n_w1;
        const int h = bias ? idx - n_w1 : idx % h_dim, i = bias ? 0 : idx / h_dim;
        const float w2h = w2_old[h];
        for (int t = 0; t < T; ++t) {
            const float hv = hidden[(size_t)t * h_dim + h];
            const float dh = __fmul_rn(__fmul_rn(dlogit[t], w2h), hv > 0.f ? 1.f : 0.f);
            g = __fadd_rn(g, bias ? dh : __fmul_rn(dh, feat[(size_t)t * in_dim + i]));
        }
        float* p = bias ? b1 + h : w1 + idx;
        *p = __fadd_rn(*p, -__fmul_rn(step, g));
    } else if (idx < n_w1 + 2 * h_dim) {    // W2[h]
        const int h = idx - n_w1 - h_dim;
        for (int t = 0; t < T; ++t) g = __fadd_rn(g, __fmul_rn(dlogit[t], hidden[(size_t)t * h_dim + h]));
        w2[h] = __fadd_rn(w2[h], -__fmul_rn(step, g));
    } else {                                // b2
        for (int t = 0; t < T; ++t) g = __fadd_rn(g, dlogit[t]);
        b2[0] = __fadd_rn(b2[0], -__fmul_rn(step, g));
    }
}

static int check_meta(const grl_kv_layout* kv, const grl_kv_meta* m) {
    GRL_REQUIRE(kv && m, "NULL argument");
    GRL_REQUIRE(kv->block_table && kv->seq_lens && kv->batch > 0 && kv->page_tokens > 0 && kv->max_pages > 0,
                "bad cache layout");
    GRL_REQUIRE(m->cum_score && m->tombstone, "NULL metadata buffer");
    GRL_REQUIRE(m->capacity >= kv->max_pages * kv->page_tokens, "metadata capacity %d below the cache's %d tokens",
                m->capacity, kv->max_pages * kv->page_tokens);
    return GRL_OK;
}

}  // namespace evict
}  // namespace grl

using namespace grl;
using namespace grl::evict;

extern "C" {

int grl_kv_score_accumulate(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, const float* attn,
                            int q_rows, int ld) {
    GRL_REQUIRE(dev, "dev is NULL");
    int rc = check_meta(kv, meta);
    if (rc) return rc;
    GRL_REQUIRE(attn && q_rows > 0 && ld > 0 && ld <= meta->capacity, "bad attention-score shape");
    DeviceGuard g(dev->ordinal);
    dim3 grid((ld + 255) / 256, kv->batch);
    score_accumulate_kernel<<<grid, 256, 0, dev->stream>>>(attn, q_rows, ld, kv->seq_lens, meta->cum_score, meta->capacity);
    GRL_LAUNCHED("score_accumulate_kernel");
    return GRL_OK;
}

int grl_kv_mass_accumulate(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, const float* scores,
                           int scores_ld, const float* partial, int num_q_heads) {
    GRL_REQUIRE(dev, "dev is NULL");
    int rc = check_meta(kv, meta);
    if (rc) return rc;
    GRL_REQUIRE(scores && partial && scores_ld > 0 && num_q_heads > 0 && num_q_heads <= 4096, "bad argument");
    GRL_REQUIRE(kv->head_dim > 0, "bad cache layout");
    DeviceGuard g(dev->ordinal);
    const int tokens = scores_ld < meta->capacity ? scores_ld : meta->capacity;
    dim3 grid((tokens + 255) / 256, kv->batch);
    mass_accumulate_kernel<<<grid, 256, 2 * num_q_heads * sizeof(float), dev->stream>>>(
        scores, scores_ld, partial, num_q_heads, kv->head_dim, kv->batch * num_q_heads, kv->seq_lens, meta->cum_score,
        meta->capacity);
    GRL_LAUNCHED("mass_accumulate_kernel");
    return GRL_OK;
}

int grl_kv_evict_lowest(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, int num_evict) {
    GRL_REQUIRE(dev, "dev is NULL");
    int rc = check_meta(kv, meta);
    if (rc) return rc;
    GRL_REQUIRE(num_evict >= 0, "num_evict must not be negative");
    DeviceGuard g(dev->ordinal);
    evict_lowest_kernel<<<kv->batch, kThreads, 0, dev->stream>>>(meta->cum_score, meta->tombstone, kv->seq_lens,
                                                                meta->capacity, num_evict);
    GRL_LAUNCHED("evict_lowest_kernel");
    return GRL_OK;
}

int grl_kv_evict_heuristic(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, float threshold) {
    GRL_REQUIRE(dev, "dev is NULL");
    int rc = check_meta(kv, meta);
    if (rc) return rc;
    DeviceGuard g(dev->ordinal);
    evict_heuristic_kernel<<<kv->batch, kThreads, 0, dev->stream>>>(meta->cum_score, meta->tombstone, meta->relevance,
                                                                   kv->seq_lens, meta->capacity, threshold);
    GRL_LAUNCHED("evict_heuristic_kernel");
    return GRL_OK;
}

int grl_kv_compact_scratch_bytes(const grl_kv_layout* kv, const grl_kv_meta* meta, size_t* bytes) {
    GRL_REQUIRE(kv && meta && bytes, "NULL argument");
    *bytes = ((size_t)kv->batch * meta->capacity + (size_t)kv->batch) * sizeof(int32_t);
    return GRL_OK;
}

int grl_kv_compact(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, void* scratch,
                   size_t scratch_bytes) {
    GRL_REQUIRE(dev, "dev is NULL");
    int rc = check_meta(kv, meta);
    if (rc) return rc;
    GRL_REQUIRE(kv->k_pages && kv->v_pages && kv->num_kv_heads > 0 && kv->head_dim > 0, "bad cache layout");
    if (kv->cache_dtype == GRL_FP8_INT4)
        return set_error(GRL_ERR_UNSUPPORTED, "compaction of a quantised (FP8 / INT4) cache is not built: its three pools have "
                                              "rows of different sizes; evict on a bf16 or fp32 cache");
    size_t need = 0;
    grl_kv_compact_scratch_bytes(kv, meta, &need);
    GRL_REQUIRE(scratch && scratch_bytes >= need, "compaction scratch too small: %zu < %zu", scratch_bytes, need);
    const int row_bytes = kv->head_dim * (kv->cache_dtype == GRL_BF16 ? 2 : 4);
    GRL_REQUIRE(row_bytes % 16 == 0 && (kMoveThreads * kMovePerThread) % (row_bytes / 16) == 0,
                "unsupported row size %d bytes", row_bytes);
    GRL_REQUIRE(((uintptr_t)kv->k_pages % 16 == 0) && ((uintptr_t)kv->v_pages % 16 == 0), "page pools must be 16-byte aligned");
    DeviceGuard g(dev->ordinal);
    int32_t* new_pos = static_cast<int32_t*>(scratch);
    int32_t* new_len = new_pos + (size_t)kv->batch * meta->capacity;
    compact_scan_kernel<<<kv->batch, kThreads, 0, dev->stream>>>(meta->tombstone, kv->seq_lens, meta->capacity, new_pos,
                                                                new_len);
    GRL_LAUNCHED("compact_scan_kernel");
    MoveArgs a{};
    a.k_pages = static_cast<uint8_t*>(kv->k_pages); a.v_pages = static_cast<uint8_t*>(kv->v_pages);
    a.block_table = kv->block_table; a.seq_lens = kv->seq_lens; a.new_pos = new_pos;
    a.Hkv = kv->num_kv_heads; a.P = kv->page_tokens; a.max_pages = kv->max_pages; a.capacity = meta->capacity;
    a.row_bytes = row_bytes;
    const int parts = row_bytes >= 256 ? 2 : 1;          // half rows of >= 128 bytes
    dim3 grid(kv->num_kv_heads, kv->batch, 2 * parts);
    compact_move_kernel<<<grid, kMoveThreads, 0, dev->stream>>>(a);
    GRL_LAUNCHED("compact_move_kernel");
    compact_meta_kernel<<<kv->batch, kThreads, 0, dev->stream>>>(meta->cum_score, meta->tombstone, meta->relevance,
                                                                kv->seq_lens, meta->evicted, new_pos, new_len,
                                                                meta->capacity);
    GRL_LAUNCHED("compact_meta_kernel");
    return GRL_OK;
}

static int check_head(const grl_evict_head* h) {
    GRL_REQUIRE(h && h->w1 && h->b1 && h->w2 && h->b2, "NULL eviction-head buffer");
    GRL_REQUIRE(h->input_dim > 0 && h->hidden_dim > 0 && h->hidden_dim <= 4096, "bad eviction-head shape");
    return GRL_OK;
}

int grl_evict_head_scratch_bytes(const grl_evict_head* head, int tokens, size_t* bytes) {
    GRL_REQUIRE(head && bytes && tokens >= 0, "bad argument");
    // received[T], dlogit[T], median[1] (+pad), hidden[T][h], w2 copy[h]
    *bytes = sizeof(float) * ((size_t)tokens * (2 + head->hidden_dim) + 4 + head->hidden_dim);
    return GRL_OK;
}

int grl_evict_head_train(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, const grl_evict_head* head,
                         const float* features, const float* attn, int seq_len, int tokens, float lr, void* scratch,
                         size_t scratch_bytes) {
    GRL_REQUIRE(dev, "dev is NULL");
    int rc = check_meta(kv, meta);
    if (!rc) rc = check_head(head);
    if (rc) return rc;
    GRL_REQUIRE(kv->batch == 1, "the eviction head works on a single-sequence cache");
    GRL_REQUIRE(meta->relevance, "metadata has no relevance array");
    GRL_REQUIRE(features && attn && seq_len > 0 && tokens > 0 && tokens <= meta->capacity, "bad argument");
    size_t need = 0;
    grl_evict_head_scratch_bytes(head, tokens, &need);
    GRL_REQUIRE(scratch && scratch_bytes >= need, "eviction-head scratch too small: %zu < %zu", scratch_bytes, need);
    DeviceGuard g(dev->ordinal);
    float* received = static_cast<float*>(scratch);
    float* dlogit = received + tokens;
    float* median = dlogit + tokens;
    float* hidden = median + 4;
    float* w2_old = hidden + (size_t)tokens * head->hidden_dim;
    const int blocks = (tokens + 127) / 128;
    head_received_kernel<<<blocks, 128, 0, dev->stream>>>(attn, seq_len, tokens, received);
    GRL_LAUNCHED("head_received_kernel");
    head_median_kernel<<<1, kThreads, 0, dev->stream>>>(received, tokens, median);
    GRL_LAUNCHED("head_median_kernel");
    HeadArgs hd{head->w1, head->b1, head->w2, head->b2, head->input_dim, head->hidden_dim};
    head_forward_kernel<<<blocks, 128, 0, dev->stream>>>(hd, features, tokens, meta->tombstone, meta->relevance, hidden,
                                                        dlogit, received, median, nullptr, 0.f);
    GRL_LAUNCHED("head_forward_kernel");
    // the W1 gradient uses W2 as it was in the forward pass, while another thread updates W2
    GRL_CUDA(cudaMemcpyAsync(w2_old, head->w2, sizeof(float) * head->hidden_dim, cudaMemcpyDeviceToDevice, dev->stream));
    const int params = head->input_dim * head->hidden_dim + 2 * head->hidden_dim + 1;
    head_update_kernel<<<(params + 127) / 128, 128, 0, dev->stream>>>(head->w1, head->b1, head->w2, head->b2,
                                                                     head->input_dim, head->hidden_dim, features, hidden,
                                                                     dlogit, w2_old, tokens, lr / (float)tokens);
    GRL_LAUNCHED("head_update_kernel");
    return GRL_OK;
}

int grl_evict_head_predict(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, const grl_evict_head* head,
                           const float* features, int tokens, float threshold) {
    GRL_REQUIRE(dev, "dev is NULL");
    int rc = check_meta(kv, meta);
    if (!rc) rc = check_head(head);
    if (rc) return rc;
    GRL_REQUIRE(kv->batch == 1, "the eviction head works on a single-sequence cache");
    GRL_REQUIRE(meta->relevance, "metadata has no relevance array");
    GRL_REQUIRE(features && tokens > 0 && tokens <= meta->capacity, "bad argument");
    DeviceGuard g(dev->ordinal);
    HeadArgs hd{head->w1, head->b1, head->w2, head->b2, head->input_dim, head->hidden_dim};
    head_forward_kernel<<<(tokens + 127) / 128, 128, 0, dev->stream>>>(hd, features, tokens, meta->tombstone, meta->relevance,
                                                                      nullptr, nullptr, nullptr, nullptr, meta->tombstone,
                                                                      threshold);
    GRL_LAUNCHED("head_forward_kernel");
    return GRL_OK;
}

}  // extern "C"

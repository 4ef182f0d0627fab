/* grilly_cuda.h -- C ABI of the B200 (sm_100a) attention path.
 *
 * This is the whole boundary between the host-side op layer (namespace grilly::ops, the
 * grilly_core pybind11 module) and the CUDA kernels.  Plain pointers and sizes only: no C++
 * types, no PyTorch types, no exceptions.  Every function returns GRL_OK (0) or a negative
 * GRL_ERR_* code; grl_last_error() gives the message of the calling thread's last failure.
 *
 * Each entry point names the piece of the reference (Grillcheese-AI/grilly-next, paths relative
 * to that project) that it replaces.
 *
 * Conventions
 *  - All data pointers are DEVICE pointers unless a parameter says "host".
 *  - All launches and copies are asynchronous on the device's stream (grl_device_use_stream
 *    adopts a caller's stream); grl_sync waits for it.
 *  - Callers own every buffer (grl_malloc / grl_free); kernels never allocate.  The library
 *    itself caches only per-device RoPE cos/sin tables (one per (head_dim, theta, scaling), sized to the
 *    longest sequence seen, rounded up to a power of two) that it frees in grl_device_close, and
 *    the encoded tensor maps of recent launches (host memory).
 */
#ifndef GRILLY_CUDA_H
#define GRILLY_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct grl_device grl_device;
typedef struct grl_event grl_event;
typedef struct grl_graph grl_graph;
typedef struct grl_group grl_group;

enum {
    GRL_OK = 0,
    GRL_ERR_INVALID = -1,     /* bad argument / shape; nothing was launched */
    GRL_ERR_CUDA = -2,        /* a CUDA runtime/driver call failed */
    GRL_ERR_UNSUPPORTED = -3, /* valid request that no kernel here covers */
    GRL_ERR_TIMEOUT = -4,     /* grl_sync host timeout, or a bounded device wait ran out */
    GRL_ERR_OOM = -5,
    GRL_ERR_KERNEL = -6       /* a kernel reported a failure through its status word */
};

enum { GRL_F32 = 0, GRL_BF16 = 1,
       GRL_FP8_INT4 = 2 /* KV cache only: FP8-E4M3 keys, INT4 values, one float16 scale per 32 key elements */ };
enum { GRL_ROPE_NONE = 0, GRL_ROPE_INTERLEAVED = 1, GRL_ROPE_HALF = 2 };
/* Mask conventions of the reference, selected by the shape the caller holds. Values > 0 keep. */
enum {
    GRL_MASK_NONE = 0,
    GRL_MASK_KEY = 1,  /* (B,S) key-padding mask: shaders/flash-attention2.glsl:151-154 */
    GRL_MASK_BSS = 2,  /* (B,S,S): the size cpp/src/ops/attention.cpp:63-66 uploads; also (B,1,S,S) */
    GRL_MASK_BHSS = 3  /* (B,H,S,S): tests/test_attention.py:29-30 */
};
enum { GRL_KERNEL_AUTO = 0, GRL_KERNEL_SIMT_F32 = 1, GRL_KERNEL_TCGEN05 = 2 };

const char* grl_last_error(void);

/* ---- device, memory, stream: replaces GrillyDevice (cpp/src/device.cpp:103-468), the VMA
 * BufferPool's allocation/upload/download (cpp/src/buffer_pool.cpp:128-175,453-477) and
 * CommandBatch submit/wait (cpp/src/command_batch.cpp:69-149). */
typedef struct {
    char name[128];
    int32_t ordinal, cc_major, cc_minor, sm_count;
    int64_t total_mem_bytes, l2_bytes, smem_per_block_optin;
} grl_device_info;

int grl_device_count(int* count);
int grl_device_open(int ordinal, grl_device** out);
int grl_device_close(grl_device* dev);
int grl_device_get_info(grl_device* dev, grl_device_info* info);
/* Launch on the caller's cudaStream_t from now on.  NULL restores the device's own (non-blocking)
 * stream; to name the legacy default stream pass cudaStreamLegacy ((cudaStream_t)0x1), since its
 * plain handle is NULL too. */
int grl_device_use_stream(grl_device* dev, void* cuda_stream);
/* Cycle budgets of the bounded waits inside the kernels; 0 restores a default.  barrier_wait_cycles
 * (default 2e9, about a second) bounds every mbarrier wait of the prefill and decode kernels;
 * peer_wait_cycles (default 1e9) bounds the wait for another GPU's partial in the cross-GPU merge
 * (grl_exchange_params.wait_cycles overrides it per call).  A wait that runs out makes the kernel
 * return; the next grl_sync reports GRL_ERR_TIMEOUT.  This is the device-side counterpart of the 2 s
 * fence timeout of cpp/src/command_batch.cpp:16,145-148. */
int grl_device_set_wait_limits(grl_device* dev, uint64_t barrier_wait_cycles, uint64_t peer_wait_cycles);
/* Lookups of encoded tensor maps by (pointer, shape, box): the role of the descriptor-set LRU of
 * PipelineCache (cpp/src/pipeline_cache.cpp:217-305).  Any pointer may be NULL. */
int grl_tensor_map_cache_stats(grl_device* dev, int64_t* hits, int64_t* misses, int64_t* cached);
int grl_malloc(grl_device* dev, size_t bytes, void** out);
int grl_free(grl_device* dev, void* ptr);
int grl_host_alloc(size_t bytes, void** out); /* pinned host memory for staging */
int grl_host_free(void* ptr);
int grl_memcpy_h2d(grl_device* dev, void* dst, const void* src_host, size_t bytes);
int grl_memcpy_d2h(grl_device* dev, void* dst_host, const void* src, size_t bytes);
int grl_memcpy_d2d(grl_device* dev, void* dst, const void* src, size_t bytes);
int grl_memset(grl_device* dev, void* dst, int value, size_t bytes);
/* Wait for the stream.  timeout_ns == 0 waits without limit; otherwise polls and returns
 * GRL_ERR_TIMEOUT when the limit passes (the 2 s fence timeout of command_batch.cpp:16,145-148). */
int grl_sync(grl_device* dev, uint64_t timeout_ns);

int grl_event_create(grl_event** out);
int grl_event_create_untimed(grl_event** out); /* ordering only (grl_event_wait): cheaper to record */
int grl_event_destroy(grl_event* ev);
int grl_event_record(grl_device* dev, grl_event* ev);
/* Work submitted to dev after this call starts only when ev (recorded on any handle's stream, of any
 * GPU) has completed; the host does not wait.  Several handles opened on one GPU are several streams:
 * this is how an upload, a kernel and a download of different chunks overlap. */
int grl_event_wait(grl_device* dev, grl_event* ev);
int grl_event_sync(grl_event* ev); /* the host waits until the event has completed */
int grl_event_elapsed_ms(grl_event* start, grl_event* stop, float* ms); /* syncs on stop */

/* Stream capture of a launch sequence (the 256-step decode loop); replaces the record-once /
 * replay role of CommandBatch + OpGraph for this path. */
int grl_graph_begin(grl_device* dev);
int grl_graph_end(grl_device* dev, grl_graph** out);
int grl_graph_launch(grl_device* dev, grl_graph* g);
int grl_graph_destroy(grl_graph* g);

/* Number of kernels this library has launched on any device since load (for accounting). */
int64_t grl_launch_count(void);

/* Element-wise dtype conversion (GRL_F32 <-> GRL_BF16, round-to-nearest-even), n elements. */
int grl_cast(grl_device* dev, const void* src, int src_dtype, void* dst, int dst_dtype, size_t n);

/* ---- prefill: replaces ops::flashAttention2 (cpp/src/ops/attention.cpp:45-166) together with
 * shaders/flash-attention2.glsl and shaders/flash-attention2-rope.glsl (push block :56-71).
 * O = softmax(rope(Q) rope(K)^T * scale, masked) V, forward only. */
typedef struct {
    const void* q;      /* (B,H,S,D) contiguous, in_dtype */
    const void* k;
    const void* v;
    void* o;            /* (B,H,S,D) contiguous, out_dtype */
    int32_t in_dtype;   /* GRL_F32 or GRL_BF16 */
    int32_t out_dtype;
    int32_t batch, heads, seq_len, head_dim;
    float scale;        /* 0 => 1/sqrt(head_dim) (attention.cpp:53-55) */
    int32_t causal;     /* key k visible to query q iff k <= q */
    const int32_t* seq_lens; /* (B) valid lengths or NULL; rows q >= len are written as 0 */
    const float* mask;  /* explicit mask or NULL */
    int32_t mask_kind;  /* GRL_MASK_* */
    int32_t rope_mode;  /* GRL_ROPE_*; position = sequence index (flash-attention2-rope.glsl:101-141) */
    float rope_theta;   /* base, e.g. 10000 */
    float rope_scaling; /* theta / scaling; 0 is read as 1 */
    int32_t kernel;     /* GRL_KERNEL_*; AUTO picks tcgen05 for bf16 input with D=128 or 64 */
    int32_t* status;    /* optional device int32[4]; [0] != 0 after a kernel-side failure */
} grl_flash_params;
int grl_flash_fwd(grl_device* dev, const grl_flash_params* p);

/* Builds (or grows) the device's cos/sin table for positions [0, n_pos) ahead of use.  grl_flash_fwd
 * does this on demand, which allocates and launches: inside a stream capture that is refused, so call
 * this first (the precomputed-table mode of shaders/rope.glsl:109-113 made implicit). */
int grl_rope_table_prepare(grl_device* dev, int n_pos, int head_dim, float theta, float scaling);

/* ---- linear projection, the step on either side of attention: replaces ops::linear (cpp/src/ops/linear.cpp:20-82,
 * shader fnn-linear) and shaders/fused-qkv-projection.glsl:40-74 (the same product with the packed
 * [W_q; W_k; W_v] weight and bias).  y (m,n) float32 = x (m,k) w^T + bias, w (n,k) row-major, bias (n) or NULL.
 * in_dtype GRL_F32: exact float32 dot products; GRL_BF16: x and w are bf16 (grl_cast) and the product runs on the
 * tcgen05 tensor cores with float32 accumulation (k must be a multiple of 8). */
int grl_linear(grl_device* dev, const void* x, const void* w, const float* bias, float* y, int m, int k, int n,
               int in_dtype);

/* ---- standalone RoPE: replaces shaders/rope.glsl:32-126 (push block :32-40).
 * x, y: (B,S,H,D) float32, out of place; position = sequence index / scaling;
 * cos_table/sin_table: optional (>=S, D/2) float32 tables (use_precomputed). */
int grl_rope(grl_device* dev, const float* x, float* y, int batch, int seq_len, int heads,
             int head_dim, float base, float scaling, int mode, const float* cos_table,
             const float* sin_table);

/* ---- standalone mask fill: replaces shaders/attention-mask.glsl:18-55.
 * scores: (B,H,S,S) float32, in place.  causal != 0: scores[k>q] = mask_value; else key_mask
 * (B,S): scores[..,k] = mask_value where key_mask[b,k] < 0.5. */
int grl_attention_mask(grl_device* dev, float* scores, const float* key_mask, int batch,
                       int heads, int seq_len, int causal, float mask_value);

/* ---- paged KV cache.  Pages are head-major: [page][Hkv][page_tokens][D] of cache_dtype, one
 * pool for K and one for V; block_table[b][i] = page holding tokens [i*page_tokens, ...) of
 * sequence b; seq_lens[b] = tokens stored.  Replaces the storage of struct KVCache
 * (cpp/include/grilly/ops/kv_cache.h:123-144) for the uncompressed mode. */
typedef struct {
    void* k_pages;
    void* v_pages;
    int32_t cache_dtype;          /* GRL_BF16 (default), GRL_F32 or GRL_FP8_INT4 */
    const int32_t* block_table;   /* (B, max_pages) */
    int32_t* seq_lens;            /* (B) */
    int32_t batch, num_kv_heads, head_dim, page_tokens, max_pages;
    int32_t num_pages;            /* pages in each pool; 0 is read as batch * max_pages */
    void* scales;                 /* GRL_FP8_INT4 only: uint16 [page][Hkv][page_tokens][head_dim/32], see below */
} grl_kv_layout;
/* GRL_FP8_INT4 is the asymmetric quantisation of the reference (cpp/src/ops/kv_cache.cpp:272-399, decode
 * :500-577), byte for byte, on the paged layout: k_pages holds one FP8-E4M3 byte per element
 * ([page][Hkv][page_tokens][D]), v_pages two INT4 codes per byte ([page][Hkv][page_tokens][D/2], even
 * element in the low nibble, stored value + 8), scales one float16 bit pattern per group of 32 key elements.
 * As in the reference only the KEY scales are kept and decode divides keys AND values by them; head_dim
 * must be a multiple of 32.  grl_kv_append quantises (after the optional RoPE of the keys), grl_kv_gather
 * dequantises, grl_gqa_decode attends over the dequantised values with the generic kernel. */

/* Append n_new tokens per sequence: replaces ops::kvCacheAppend (cpp/src/ops/kv_cache.cpp:155-419;
 * signature kv_cache.h:163-166) and fuses the RoPE of the new keys and of the step's queries.
 * k_new, v_new: (B, n_new, Hkv, D) float32.  q_in/q_out: optional (B, n_new, Hq, D) float32,
 * rotated at the same positions (position = pos_base + seq_lens[b] + i).  update_lens != 0
 * adds n_new to seq_lens[b] afterwards. */
typedef struct {
    grl_kv_layout kv;
    const float* k_new;
    const float* v_new;
    const float* q_in;
    float* q_out;
    int32_t n_new, num_q_heads;
    int32_t rope_mode;
    float rope_theta, rope_scaling;
    int32_t pos_base;
    int32_t update_lens;
    const int32_t* pos_offsets; /* optional device int32[B]: added to the position of sequence b (the tokens
                                 * compaction has removed from it, grl_kv_meta.evicted) */
} grl_append_params;
int grl_kv_append(grl_device* dev, const grl_append_params* p);

/* Materialise sequence b as token-major float32 (T, Hkv, D): replaces ops::kvCacheDecode
 * (cpp/src/ops/kv_cache.cpp:435-578; kv_cache.h:175-177). */
int grl_kv_gather(grl_device* dev, const grl_kv_layout* kv, int b, int n_tokens, float* out_k,
                  float* out_v);

/* ---- MLA latent path of the KV cache (cpp/src/ops/kv_cache.cpp:174-248 compress, :441-498 decode).
 * grl_gemm_f32: C (m,n) = A (m,k) B (k,n), row-major float32: replaces the gemm_mnk shader those paths dispatch
 * (shaders/gemm_mnk.glsl:34-80; sum over k ascending, unfused multiply and add).
 * grl_mla_concat / grl_mla_split: (rows, D) K and V <-> (rows, 2D) [K | V] rows, the host loops around the two
 * projections (:190-203, :483-494). */
int grl_gemm_f32(grl_device* dev, const float* a, const float* b, float* c, int m, int k, int n);
int grl_mla_concat(grl_device* dev, const float* k, const float* v, float* out, size_t rows, int head_dim);
int grl_mla_split(grl_device* dev, const float* in, float* k, float* v, size_t rows, int head_dim);

/* Block swizzle of a (B,H,S,D) float32 tensor into (B,H,ceil(S/W),ceil(D/W),W,W) with zero padding, or
 * back (reverse != 0): replaces ops::swizzle / swizzleCPU / unswizzleCPU (cpp/src/ops/swizzle.cpp:49-229).
 * The swizzled side holds B*H*S_pad*D_pad floats. */
int grl_swizzle_kv(grl_device* dev, const float* in, float* out, int batch, int heads, int seq_len, int head_dim,
                   int wave, int reverse);

/* ---- the unfused attention pieces (float32, device pointers), for code written against the separate shaders.
 * grl_attention_scores: scores (B,H,S,S) = scale * Q K^T with Q, K laid out (B,S,H,D): replaces
 *   shaders/attention-scores.glsl:33-65.  scale 0 means 1/sqrt(D).
 * grl_softmax: row-wise softmax over the last axis of (rows, features): replaces shaders/activation-softmax.glsl:34-84
 *   (its three passes in one launch; the maximum starts from -1e10 as the shader's does).
 * grl_attention_output: out (B,S,H,D) = weights (B,H,S,S) . V (B,S,H,D): replaces shaders/attention-output.glsl:28-70
 *   (causal == 0) and shaders/attention-output-gpt.glsl:29-72 (causal != 0: the sum runs over k <= q only).
 * grl_attention_backward: gradients of softmax(scale Q K^T) V given grad_out and the forward's weights, every
 *   tensor (B,H,S,D) and attn / scratch (B,H,S,S): replaces the three passes of shaders/attention-backward.glsl:73-195
 *   (grad_V = A^T gO; grad_A = gO V^T into scratch; softmax backward; grad_Q = scale gS K; grad_K = scale gS^T Q)
 *   and VulkanBackwardOps.attention_backward (src/grilly_next/backend/autograd_core.py:617-655). */
int grl_attention_scores(grl_device* dev, const float* q, const float* k, float* scores, int batch, int seq_len, int heads,
                         int head_dim, float scale);
int grl_softmax(grl_device* dev, const float* in, float* out, size_t rows, int features);
int grl_attention_output(grl_device* dev, const float* weights, const float* v, float* out, int batch, int seq_len,
                         int heads, int head_dim, int causal);
int grl_attention_backward(grl_device* dev, const float* grad_out, const float* q, const float* k, const float* v,
                           const float* attn, float* grad_q, float* grad_k, float* grad_v, float* scratch, int batch,
                           int heads, int seq_len, int head_dim, float scale);

/* ---- eviction on the paged cache: replaces the host loops of kvCacheEvictH2O
 * (cpp/src/ops/kv_cache.cpp:595-634), the untrained-head branch of kvCacheEvictSpeculative (:905-929)
 * and kvCacheCompact (:941-992; signatures kv_cache.h:186-229).  The reference's TokenMeta array
 * (kv_cache.h:68-73) becomes device arrays, one entry per token slot of every sequence; all-zero is
 * the state of a fresh cache, and appended tokens need no initialisation. */
typedef struct {
    float* cum_score;     /* [B][capacity] attention mass received so far (TokenMeta.cumulativeScore) */
    uint8_t* tombstone;   /* [B][capacity] 1 = evicted, awaiting compaction (nextActive == UINT32_MAX-1) */
    float* relevance;     /* [B][capacity] TokenMeta.predictedRelevance; may be NULL */
    int32_t* evicted;     /* [B] tokens compaction has removed from the sequence; may be NULL */
    int32_t capacity;     /* token slots per sequence, >= max_pages * page_tokens */
} grl_kv_meta;
/* cum_score[b][t] += sum over q of attn[b][q][t], t < seq_lens[b]; attn is (B, q_rows, ld) float32
 * probabilities.  The sum runs in ascending q with float adds, as kv_cache.cpp:606-615 does. */
int grl_kv_score_accumulate(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta,
                            const float* attn, int q_rows, int ld);
/* One decode step's contribution without an attention matrix from the caller: cum_score[b][t] +=
 * sum over the Hq query heads of softmax probability p[b][h][t] = exp(scores[b][h][t] - m[b][h]) / l[b][h],
 * with `scores` the scores_out of grl_gqa_decode and `partial` its partial_out ([O | m | l]) of the same
 * call.  Heads add in ascending order. */
int grl_kv_mass_accumulate(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, const float* scores,
                           int scores_ld, const float* partial, int num_q_heads);
/* Tombstone the num_evict tokens with the lowest cum_score in every sequence (0 => a quarter of the
 * sequence; nothing happens where num_evict >= its length).  Ties go to the lowest index. */
int grl_kv_evict_lowest(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, int num_evict);
/* relevance = 0.7 * cum_score / max(cum_score) + 0.3 * t / len; tombstone where it is below threshold. */
int grl_kv_evict_heuristic(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, float threshold);
/* Move the live tokens of every sequence to the front (order kept, K and V rows and scores), clear the
 * tombstones, shrink seq_lens, add the removed count to meta->evicted.  scratch: device memory of
 * grl_kv_compact_scratch_bytes(). */
int grl_kv_compact_scratch_bytes(const grl_kv_layout* kv, const grl_kv_meta* meta, size_t* bytes);
int grl_kv_compact(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, void* scratch,
                   size_t scratch_bytes);

/* Trainable eviction head (kvCacheTrainEvictionHead, cpp/src/ops/kv_cache.cpp:734-845, and the
 * trained-head branch of kvCacheEvictSpeculative, :856-903): relevance = sigmoid(W2 . relu(W1^T x + b1) + b2)
 * per token of a single-sequence cache.  w1 (input_dim, hidden_dim) row-major, b1 (hidden_dim),
 * w2 (hidden_dim), b2 (1): device float32, owned and initialised by the caller. */
typedef struct {
    float* w1;
    float* b1;
    float* w2;
    float* b2;
    int32_t input_dim, hidden_dim;
} grl_evict_head;
int grl_evict_head_scratch_bytes(const grl_evict_head* head, int tokens, size_t* bytes);
/* One SGD step: labels = (attention received > its median), attention received = column sums of attn
 * (seq_len, tokens); binary cross-entropy; mean gradient over `tokens`; tombstoned tokens are skipped.
 * features (tokens, input_dim), attn: device float32.  Writes the predictions to meta->relevance. */
int grl_evict_head_train(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, const grl_evict_head* head,
                         const float* features, const float* attn, int seq_len, int tokens, float lr, void* scratch,
                         size_t scratch_bytes);
/* Predict relevance of every live token and tombstone those below threshold. */
int grl_evict_head_predict(grl_device* dev, const grl_kv_layout* kv, const grl_kv_meta* meta, const grl_evict_head* head,
                           const float* features, int tokens, float threshold);

/* ---- decode attention: replaces shaders/gqa-attention.glsl:34-130 (no host dispatcher exists
 * in the reference).  q, out: (B,1,Hq,D) float32.  kv_head = q_head / (Hq/Hkv).
 * The KV range of every sequence is cut into n_splits parts that run on different SMs; each
 * part leaves (O un-normalised, m, l) in `workspace`, and a merge pass combines them.
 * If partial_out != NULL the merged result is written there UN-normalised as
 * [O (B*Hq*D) | m (B*Hq) | l (B*Hq)] floats (one part of a cross-GPU merge) and `out` may be NULL. */
typedef struct {
    grl_kv_layout kv;
    const float* q;
    float* out;
    int32_t num_q_heads;
    float scale;            /* 0 => 1/sqrt(D) */
    int32_t n_splits;       /* 0 => chosen from max_seq_len and the SM count */
    int32_t max_seq_len;    /* upper bound of seq_lens (host knowledge; sizes the split) */
    void* workspace;        /* >= grl_decode_workspace_bytes() */
    size_t workspace_bytes;
    float* partial_out;
    int32_t force_simt;     /* != 0: use the generic SIMT kernel even where the tensor-core path applies */
    float* scores_out;      /* optional (B*Hq, scores_ld) float32: the scaled scores q.k of every cached token,
                             * natural-log domain, written for t < seq_lens[b] (what H2O eviction accumulates:
                             * grl_kv_mass_accumulate) */
    int32_t scores_ld;
    const struct grl_exchange_params_s* exchange;   /* optional, see grl_exchange_params below: the KV shards of
                             * other GPUs are merged in over NVLink inside the decode kernel; `out` then holds
                             * the attention over ALL ranks' shards.  NULL: single-GPU decode. */
} grl_decode_params;
int grl_decode_pick_splits(grl_device* dev, const grl_decode_params* p, int* n_splits);
int grl_decode_workspace_bytes(const grl_decode_params* p, int n_splits, size_t* bytes);
int grl_gqa_decode(grl_device* dev, const grl_decode_params* p);

/* The same decode step for callers that cannot allocate device memory and cannot pass a workspace
 * (a process whose own arena owns all device memory after start-up, a plugin that only ever
 * receives its input and output tensors).  This entry point has no counterpart in the reference.
 * The split-KV partials go to a 4 MiB array that is part of the library's device image (each GPU
 * that loads the library holds it until exit); p->workspace / workspace_bytes are ignored.
 * Returns GRL_ERR_INVALID, launching nothing, when n_splits * batch * num_q_heads * (head_dim + 2)
 * floats exceed 4 MiB.  No cudaMalloc / cudaFree / allocating routine is called.
 * - The first call on a device looks up the array's device address; make that call before any
 *   stream capture.
 * - All calls share the one array, which keeps the previous call's contents.  Nothing in it has to
 *   start at zero (every partial is fully written before it is read), but two calls that overlap
 *   on the GPU (different streams, different devices' handles on one GPU) race on it. */
int grl_gqa_decode_static(grl_device* dev, const grl_decode_params* p);

/* Log-sum-exp merge of n_parts partials laid out as the partial_out of grl_gqa_decode, part i at
 * parts + i*part_stride floats.  rows = B*Hq.  normalise != 0 writes O/l to out (rows*D);
 * otherwise writes one combined partial of the same layout to out. */
int grl_lse_merge(grl_device* dev, const float* parts, int n_parts, size_t part_stride, int rows,
                  int head_dim, int normalise, float* out);

/* ---- cross-GPU merge over NVLink peer memory (one process per GPU).  No counterpart in the
 * reference, which has no multi-GPU code; it is the exchange step of the KV-sharded decode.
 * grl_ipc_export / grl_ipc_import / grl_ipc_release wrap the CUDA IPC handle (64 bytes) of a
 * grl_malloc'ed buffer so that ranks can map one another's inboxes.
 * grl_exchange_merge: stores this rank's partial (layout of grl_gqa_decode's partial_out, n =
 * rows*(head_dim+2) floats) into every peer's inbox, waits -- at most wait_cycles (default ~0.5 s), then
 * GRL_ERR_TIMEOUT through grl_sync -- for the peers' partials of the same step, and writes the
 * normalised merge to out.  After a timeout the ranks' step counters may differ (a rank that gave up
 * has counted the step, the exchange inside the decode kernel has not): every rank then calls
 * grl_exchange_reset, which zeroes its inbox, flags and step counter, and the ranks meet at a host
 * barrier before the next step.  inbox: local float[2][world][n]; flags: local uint32[2][world], zero before the first step;
 * seq: local uint32 step counter, zero before the first step (the call increments it on the
 * device, so a captured CUDA graph can be replayed); peer_inbox / peer_flags: HOST arrays of
 * `world` device pointers (imported; the entry of this rank is ignored).  Every rank must make the
 * same sequence of calls.
 * With flag_slots = S the flags are uint32[2][world][S]; grl_exchange_merge uses slot 0.
 * grl_decode_params.exchange (tensor-core geometry only: bf16 cache at head_dim 128 or 64, or the quantised cache
 * at 128; pages of 64, 32 or 16 tokens; B*Hkv <= the SM count; low_latency inbox format) goes one step further: the CTA that finishes a (sequence, kv
 * head) last merges its splits, stores the head's rows into the peers' inboxes, waits for theirs and
 * writes the final rows -- decode, exchange and merge are ONE launch per step; local_partial, out,
 * rows and head_dim of the exchange struct are then ignored. */
typedef struct grl_exchange_params_s {
    const float* local_partial;
    float* inbox;
    uint32_t* flags;
    float* const* peer_inbox;
    uint32_t* const* peer_flags;
    uint32_t* seq;
    float* out;
    int32_t rank, world, rows, head_dim;
    int32_t flag_slots;     /* flags per (parity, peer); 0 is read as 1 */
    int32_t low_latency;    /* != 0 => every inbox element is 8 bytes {value, step number}
                             * (inbox: uint2[2][world][n], twice the bytes, zero before the first step); the flags
                             * are not used and no fence separates data from flag: one NVLink crossing per step */
    uint64_t wait_cycles;   /* cycle budget of the wait for the peers; 0 => the device's peer_wait_cycles */
} grl_exchange_params;
int grl_ipc_export(grl_device* dev, void* ptr, void* handle_out_64_bytes);
int grl_ipc_import(grl_device* dev, const void* handle_64_bytes, void** ptr_out);
int grl_ipc_release(grl_device* dev, void* ptr);
int grl_exchange_merge(grl_device* dev, const grl_exchange_params* p);
int grl_exchange_reset(grl_device* dev, const grl_exchange_params* p);

/* ---- NCCL communicator, one process per GPU.  No counterpart in the reference (it has no communication
 * backend); this is the collective form of the exchange step above: all-gather of the partials over
 * NVLink/NVSwitch, then the log-sum-exp merge.  libnccl.so.2 is opened at run time; without it these entry
 * points return GRL_ERR_UNSUPPORTED and everything else works.
 * grl_group_unique_id: rank 0 makes the 128-byte id and hands it to the other ranks by any host channel.
 * grl_group_init_rank: collective; the group launches on dev's stream.
 * grl_group_allgather_merge: partial = this rank's [O | m | l] (rows*(head_dim+2) floats), gather_buf =
 * world times that, out = (rows, head_dim) normalised.  timeout_ns == 0 only enqueues (stream order; a CUDA
 * graph can capture it); otherwise the call waits like grl_group_sync.
 * grl_group_sync: waits for the stream while polling ncclCommGetAsyncError; a remote failure or the time limit
 * aborts the communicator (ncclCommAbort) and returns an error; the group is then only good for
 * grl_group_destroy. */
int grl_group_unique_id(void* id_out_128_bytes);
int grl_group_init_rank(grl_device* dev, const void* id_128_bytes, int rank, int world, grl_group** out);
int grl_group_info(grl_group* group, int* rank, int* world, int* nccl_version);
int grl_group_allgather(grl_group* group, const void* send, void* recv, size_t bytes_per_rank);
int grl_group_allreduce_max_f64(grl_group* group, double* inout_device, size_t n);
int grl_group_allgather_merge(grl_group* group, const float* partial, int rows, int head_dim, float* gather_buf,
                              float* out, uint64_t timeout_ns);
int grl_group_sync(grl_group* group, uint64_t timeout_ns);
int grl_group_destroy(grl_group* group);

#ifdef __cplusplus
}
#endif
#endif /* GRILLY_CUDA_H */

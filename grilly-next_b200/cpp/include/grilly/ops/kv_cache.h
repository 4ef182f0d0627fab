#pragma once
// Paged, head-major KV cache and GQA decode.  Keeps the reference's KV-cache op surface
// (cpp/include/grilly/ops/kv_cache.h:46-65,123-177,232-240) for the uncompressed mode
// (compressionRatio == 1, no quantisation), in which the reference stores only metadata; here
// the tokens are stored, in pages [page][Hkv][pageTokens][D] of bf16 (or float32).
#include <cstdint>
#include <vector>

#include "grilly/buffer_pool.h"
#include "grilly/command_batch.h"
#include "grilly/ops/attention.h"
#include "grilly/pipeline_cache.h"

namespace grilly {
namespace ops {

struct KVCacheConfig {
    // reference fields (kv_cache.h:46-65)
    uint32_t maxSeqLen = 2048;
    uint32_t numHeads = 8;            // KV heads
    uint32_t headDim = 64;
    uint32_t numLayers = 12;
    uint32_t compressionRatio = 1;    // > 1: MLA latents of headDim / ratio per (token, head) instead of pages
    uint32_t maxCacheTokens = 2048;   // capacity per sequence
    bool useAsymmetricQuant = false;  // FP8-E4M3 keys + INT4 values + float16 group scales (kv_cache.cpp:250-400 there)
    uint32_t valueBits = 4;
    bool crossLayerSharing = false;
    bool useH2O = false;              // append beyond maxCacheTokens evicts the lowest-scoring tokens first
    bool useSpeculativeEviction = false;
    float evictionThreshold = 0.1f;
    // paged-cache additions
    uint32_t batchSize = 1;           // sequences held
    uint32_t pageTokens = 64;
    int dtype = GRL_BF16;             // storage type of the pages (useAsymmetricQuant overrides it with GRL_FP8_INT4)
};

/// Trainable auxiliary head for speculative eviction (the reference's EvictionHead, kv_cache.h:100-121;
/// its gradient buffers are not needed: the update kernel reduces and applies a gradient in one pass).
struct EvictionHead {
    GrillyBuffer w1, b1, w2, b2;      // (inputDim, hiddenDim), (hiddenDim), (hiddenDim), (1): float32 in HBM
    uint32_t inputDim = 0, hiddenDim = 0;
    float learningRate = 1e-3f;
    uint32_t totalUpdates = 0;
    bool initialized = false;
    grl_evict_head view() const;
};

struct KVCache {
    GrillyBuffer kPages, vPages;      // [numPages][Hkv][pageTokens][D]
    GrillyBuffer scales;              // quantised cache: float16 bits [numPages][Hkv][pageTokens][D/32]
    // MLA mode (compressionRatio > 1, single sequence; cpp/src/ops/kv_cache.cpp:64-82,174-248,441-498 there): the
    // cache keeps latents = [K | V] W_down per (token, head) and decodes [K | V] = latents W_up.  kPages then
    // aliases `latents` (no pages exist).  The reference never initialises its two matrices; here they start
    // as zeros and kvCacheSetMLAWeights sets them.
    GrillyBuffer wDown, wUp, latents; // (2D, L), (L, 2D), (maxCacheTokens, H, L) float32
    uint32_t latentDim = 0;
    bool mla() const { return latentDim != 0; }
    GrillyBuffer blockTable;          // int32 [B][maxPages]
    GrillyBuffer seqLens;             // int32 [B]
    std::vector<int32_t> hostBlockTable;
    std::vector<int32_t> hostSeqLens; // host mirror (lengths advance deterministically)
    uint32_t maxPages = 0;            // per sequence
    uint32_t numPages = 0;            // in the pool
    uint32_t nextFreePage = 0;        // bump allocator over the pool (no eviction => no free list churn)
    uint32_t currentLen = 0;          // tokens of sequence 0 (the reference's single-sequence view)
    uint64_t totalAppended = 0;
    uint64_t totalEvicted = 0;        // tokens removed by compaction, all sequences
    // Per-token metadata of the eviction family (the reference's TokenMeta array, kv_cache.h:68-73), in HBM:
    GrillyBuffer cumScore;            // float  [B][capacity]
    GrillyBuffer tombstone;           // uint8  [B][capacity]
    GrillyBuffer relevance;           // float  [B][capacity]
    GrillyBuffer evicted;             // int32  [B]: tokens compaction removed (RoPE position offset of appends)
    grl_device* device = nullptr;     // the device the buffers live on (stats read the metadata back)
    EvictionHead evictionHead;
    uint32_t capacity() const { return maxPages * config.pageTokens; }
    grl_kv_meta meta() const;
    KVCacheConfig config;
    grl_kv_layout layout() const;
};

struct KVCacheStats {
    uint32_t currentTokens, maxTokens, totalEvicted, totalAppended;
    float compressionRatio, avgAttentionScore;
    uint32_t pagesTotal, pagesUsed;
    uint64_t bytes;
};

KVCache createKVCache(BufferPool& pool, const KVCacheConfig& config);
void destroyKVCache(BufferPool& pool, KVCache& cache);

/// Reference form (kv_cache.h:163-166): newKeys/newValues (numNewTokens, numHeads, headDim) host
/// float32, appended to sequence 0 (batchSize 1) -- or (B, numNewTokens, numHeads, headDim) when
/// the cache holds B sequences.  No RoPE.
void kvCacheAppend(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, KVCache& kvCache,
                   const float* newKeys, const float* newValues, uint32_t numNewTokens);

/// Append with fused RoPE of the new keys (and optionally of the step's queries, rotated in place
/// into qOut) at position posBase + current length.
void kvCacheAppendRope(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, KVCache& kvCache,
                       const float* newKeys, const float* newValues, uint32_t numNewTokens, const float* qIn,
                       float* qOut, uint32_t numQHeads, RopeMode mode, float theta, float scaling,
                       int32_t posBase = 0);

/// Reference form (kv_cache.h:175-177): sequence `seq` back as (T, numHeads, headDim) float32.
void kvCacheDecode(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const KVCache& kvCache,
                   float* decodedKeys, float* decodedValues, uint32_t seq = 0);

KVCacheStats kvCacheGetStats(const KVCache& kvCache);

/// MLA projection matrices from the host: wDown (2*headDim, latentDim), wUp (latentDim, 2*headDim), row-major.
void kvCacheSetMLAWeights(BufferPool& pool, KVCache& kvCache, const float* wDown, const float* wUp);

/// GQA decode attention over the cache (shaders/gqa-attention.glsl:34-130): q, out (B,1,Hq,D)
/// host float32, already rotated.  accumulateScores: also add the attention mass every cached token
/// received in this step (summed over the query heads) to its cumulative score, the quantity
/// kvCacheEvictH2O ranks by -- without the caller having to build an attention matrix.
void gqaAttention(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const KVCache& kvCache,
                  const float* q, float* out, uint32_t numQHeads, float scale = 0.0f, int nSplits = 0,
                  bool accumulateScores = false);

/// One decode step: RoPE(q, k) at the current position, append k/v, attend over the cache.
/// q (B,1,Hq,D), kNew/vNew (B,1,Hkv,D), out (B,1,Hq,D): host float32.
void decodeStep(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, KVCache& kvCache, const float* q,
                const float* kNew, const float* vNew, float* out, uint32_t numQHeads, RopeMode mode, float theta,
                float scaling, float scale = 0.0f, bool accumulateScores = false);

/// Device-resident forms: q / kNew / vNew / out are HBM float32 buffers; asynchronous on the context
/// stream (no copy, no wait).  `ws` receives the pooled split-KV workspace, to be released by the
/// caller once the stream has passed the launch.
void gqaAttentionDevice(BufferPool& pool, PipelineCache& cache, const KVCache& kvCache, const GrillyBuffer& q,
                        GrillyBuffer& out, uint32_t numQHeads, float scale, int nSplits, GrillyBuffer& ws);
void decodeStepDevice(BufferPool& pool, PipelineCache& cache, KVCache& kvCache, const GrillyBuffer& q,
                      const GrillyBuffer& kNew, const GrillyBuffer& vNew, GrillyBuffer& qRotated, GrillyBuffer& out,
                      uint32_t numQHeads, RopeMode mode, float theta, float scaling, float scale, GrillyBuffer& ws);

// Eviction family of the reference (kv_cache.h:186-229) on the paged cache.
/// attentionScores: nullptr, or host (T, T) probabilities of sequence 0 -- (B, T, T) for a batched cache
/// with every sequence at length T -- whose column sums are added to the cumulative scores first
/// (kv_cache.cpp:603-616).  Then the numEvict lowest-scoring tokens of every sequence are tombstoned
/// (0 => a quarter; nothing where numEvict >= the length).  Ties go to the lowest index.
void kvCacheEvictH2O(CommandBatch&, BufferPool&, PipelineCache&, KVCache&, const float* attentionScores,
                     uint32_t numEvict = 0);
/// Eviction head: Xavier-uniform weights drawn with rand() as the reference draws them (kv_cache.cpp:653-701),
/// one SGD step on binarised attention (:734-845).  Single-sequence caches only.
void kvCacheInitEvictionHead(BufferPool& pool, KVCache& kvCache, uint32_t inputDim, uint32_t hiddenDim = 32,
                             float lr = 1e-3f);
void kvCacheDestroyEvictionHead(BufferPool& pool, KVCache& kvCache);
/// tokenFeatures (currentLen, inputDim), attentionScores (seqLen, currentLen): host float32.
void kvCacheTrainEvictionHead(CommandBatch&, BufferPool&, PipelineCache&, KVCache&, const float* tokenFeatures,
                              const float* attentionScores, uint32_t seqLen);
/// With a trained head and hiddenStates (currentLen, head.inputDim): predicted relevance below
/// config.evictionThreshold tombstones the token (kv_cache.cpp:863-903).  Otherwise the heuristic
/// (:905-929): relevance = 0.7 cum/max + 0.3 t/len.
void kvCacheEvictSpeculative(CommandBatch&, BufferPool&, PipelineCache&, KVCache&, const float* hiddenStates,
                             uint32_t hiddenDim);
/// Move live tokens to the front of every sequence and shrink the lengths (kv_cache.cpp:941-992).
void kvCacheCompact(CommandBatch&, BufferPool&, PipelineCache&, KVCache&);
/// Metadata of sequence `seq` back on the host: cumulative scores, tombstones, predicted relevance.
void kvCacheTokenMeta(BufferPool& pool, const KVCache&, uint32_t seq, std::vector<float>& cumScore,
                      std::vector<uint8_t>& tombstone, std::vector<float>& relevance);

}  // namespace ops
}  // namespace grilly

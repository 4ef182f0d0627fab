// Host side of the paged KV cache and the GQA decode ops.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>

#include "grilly/ops/kv_cache.h"

namespace grilly {
namespace ops {

namespace {
size_t elemSize(int dtype) { return dtype == GRL_BF16 ? 2 : 4; }

struct Recording {
    CommandBatch& batch;
    explicit Recording(CommandBatch& b) : batch(b) { batch.begin(); }
    ~Recording() {
        if (batch.recording()) batch.submitNoWait();
    }
};

// Give every sequence pages for `extra` more tokens; uploads the block table when it changed.
void reservePages(BufferPool& pool, KVCache& kv, uint32_t extra) {
    const auto& c = kv.config;
    bool changed = false;
    for (uint32_t b = 0; b < c.batchSize; ++b) {
        const uint32_t need = (uint32_t(kv.hostSeqLens[b]) + extra + c.pageTokens - 1) / c.pageTokens;
        if (need > kv.maxPages)
            throw std::runtime_error("kvCacheAppend: sequence would exceed max_cache_tokens (" +
                                     std::to_string(c.maxCacheTokens) + ")");
        for (uint32_t i = 0; i < need; ++i) {
            int32_t& slot = kv.hostBlockTable[size_t(b) * kv.maxPages + i];
            if (slot < 0) {
                if (kv.nextFreePage >= kv.numPages) throw std::runtime_error("kvCacheAppend: page pool exhausted");
                slot = int32_t(kv.nextFreePage++);
                changed = true;
            }
        }
    }
    if (changed) {
        // unassigned entries are uploaded as page 0; they are never read (beyond seq_lens)
        std::vector<int32_t> tmp(kv.hostBlockTable);
        for (auto& x : tmp) x = std::max(x, 0);
        // synchronous: the staging vector dies at scope exit
        check(grl_memcpy_h2d(pool.device().handle(), kv.blockTable.dptr, tmp.data(), tmp.size() * 4),
              "kvCache: block table upload");
        check(grl_sync(pool.device().handle(), 0), "kvCache: block table upload");
    }
}
}  // namespace

grl_kv_layout KVCache::layout() const {
    grl_kv_layout l{};
    l.k_pages = kPages.dptr;
    l.v_pages = vPages.dptr;
    l.cache_dtype = config.dtype;
    l.block_table = static_cast<const int32_t*>(blockTable.dptr);
    l.seq_lens = static_cast<int32_t*>(seqLens.dptr);
    l.batch = int(config.batchSize);
    l.num_kv_heads = int(config.numHeads);
    l.head_dim = int(config.headDim);
    l.page_tokens = int(config.pageTokens);
    l.max_pages = int(maxPages);
    l.num_pages = int(numPages);
    l.scales = scales.dptr;
    return l;
}

grl_kv_meta KVCache::meta() const {
    grl_kv_meta m{};
    m.cum_score = static_cast<float*>(cumScore.dptr);
    m.tombstone = static_cast<uint8_t*>(tombstone.dptr);
    m.relevance = static_cast<float*>(relevance.dptr);
    m.evicted = static_cast<int32_t*>(evicted.dptr);
    m.capacity = int32_t(capacity());
    return m;
}

KVCache createKVCache(BufferPool& pool, const KVCacheConfig& cfg) {
    if (cfg.compressionRatio == 0) throw std::runtime_error("createKVCache: compression_ratio must be at least 1");
    if (cfg.numHeads == 0 || cfg.headDim == 0 || cfg.batchSize == 0 || cfg.pageTokens == 0 || cfg.maxCacheTokens == 0)
        throw std::runtime_error("createKVCache: empty shape");
    if (cfg.headDim != 32 && cfg.headDim != 64 && cfg.headDim != 128)
        throw std::runtime_error("createKVCache: head_dim must be 32, 64 or 128");
    if (cfg.dtype != GRL_BF16 && cfg.dtype != GRL_F32 && cfg.dtype != GRL_FP8_INT4)
        throw std::runtime_error("createKVCache: unknown dtype");
    KVCache kv;
    kv.config = cfg;
    const bool quant = cfg.useAsymmetricQuant || cfg.dtype == GRL_FP8_INT4;
    if (quant) {
        if (cfg.valueBits != 4) throw std::runtime_error("createKVCache: the quantised cache stores 4-bit values (value_bits=4)");
        kv.config.dtype = GRL_FP8_INT4;
        kv.config.useAsymmetricQuant = true;
    }
    kv.maxPages = (cfg.maxCacheTokens + cfg.pageTokens - 1) / cfg.pageTokens;
    kv.numPages = kv.maxPages * cfg.batchSize;
    if (cfg.compressionRatio > 1) {
        // MLA latents (kv_cache.cpp:64-82): one sequence, float32, no pages
        if (cfg.batchSize != 1) throw std::runtime_error("createKVCache: the MLA latent cache holds one sequence (batch_size=1)");
        if (cfg.headDim % cfg.compressionRatio != 0)
            throw std::runtime_error("createKVCache: head_dim must be a multiple of compression_ratio");
        if (quant) throw std::runtime_error("createKVCache: quantised storage goes with compression_ratio=1");
        kv.latentDim = cfg.headDim / cfg.compressionRatio;
        kv.config.dtype = GRL_F32;
        const size_t w = size_t(2) * cfg.headDim * kv.latentDim * 4;
        kv.wDown = pool.acquire(w);
        kv.wUp = pool.acquire(w);
        kv.latents = pool.acquire(size_t(kv.capacity()) * cfg.numHeads * kv.latentDim * 4);
        kv.kPages = kv.latents;
        check(grl_memset(pool.device().handle(), kv.wDown.dptr, 0, w), "createKVCache");
        check(grl_memset(pool.device().handle(), kv.wUp.dptr, 0, w), "createKVCache");
        kv.numPages = 0;
    } else if (quant) {
        // one key byte and half a value byte per element, one float16 scale per group of 32 key elements
        const size_t rows = size_t(cfg.numHeads) * cfg.pageTokens * kv.numPages;
        kv.kPages = pool.acquire(rows * cfg.headDim);
        kv.vPages = pool.acquire(rows * cfg.headDim / 2);
        kv.scales = pool.acquire(rows * (cfg.headDim / 32) * 2);
    } else {
        const size_t pageBytes = size_t(cfg.numHeads) * cfg.pageTokens * cfg.headDim * elemSize(cfg.dtype);
        kv.kPages = pool.acquire(pageBytes * kv.numPages);
        kv.vPages = pool.acquire(pageBytes * kv.numPages);
    }
    kv.blockTable = pool.acquire(size_t(kv.maxPages) * cfg.batchSize * 4);
    kv.seqLens = pool.acquire(size_t(cfg.batchSize) * 4);
    kv.hostBlockTable.assign(size_t(kv.maxPages) * cfg.batchSize, -1);
    kv.hostSeqLens.assign(cfg.batchSize, 0);
    grl_device* dev = pool.device().handle();
    kv.device = dev;
    const size_t slots = size_t(kv.capacity()) * cfg.batchSize;
    kv.cumScore = pool.acquire(slots * 4);
    kv.tombstone = pool.acquire(slots);
    kv.relevance = pool.acquire(slots * 4);
    kv.evicted = pool.acquire(size_t(cfg.batchSize) * 4);
    check(grl_memset(dev, kv.cumScore.dptr, 0, slots * 4), "createKVCache");
    check(grl_memset(dev, kv.tombstone.dptr, 0, slots), "createKVCache");
    check(grl_memset(dev, kv.relevance.dptr, 0, slots * 4), "createKVCache");
    check(grl_memset(dev, kv.evicted.dptr, 0, size_t(cfg.batchSize) * 4), "createKVCache");
    check(grl_memset(dev, kv.blockTable.dptr, 0, size_t(kv.maxPages) * cfg.batchSize * 4), "createKVCache");
    check(grl_memset(dev, kv.seqLens.dptr, 0, size_t(cfg.batchSize) * 4), "createKVCache");
    check(grl_sync(dev, 0), "createKVCache");
    return kv;
}

grl_evict_head EvictionHead::view() const {
    grl_evict_head v{};
    v.w1 = static_cast<float*>(w1.dptr); v.b1 = static_cast<float*>(b1.dptr);
    v.w2 = static_cast<float*>(w2.dptr); v.b2 = static_cast<float*>(b2.dptr);
    v.input_dim = int32_t(inputDim); v.hidden_dim = int32_t(hiddenDim);
    return v;
}

void destroyKVCache(BufferPool& pool, KVCache& kv) {
    kvCacheDestroyEvictionHead(pool, kv);
    if (kv.mla()) {
        kv.kPages = GrillyBuffer{};       // an alias of `latents`
        pool.release(kv.wDown);
        pool.release(kv.wUp);
        pool.release(kv.latents);
        kv.latentDim = 0;
    }
    pool.release(kv.kPages);
    pool.release(kv.vPages);
    pool.release(kv.scales);
    pool.release(kv.blockTable);
    pool.release(kv.seqLens);
    pool.release(kv.cumScore);
    pool.release(kv.tombstone);
    pool.release(kv.relevance);
    pool.release(kv.evicted);
    kv.hostBlockTable.clear();
    kv.hostSeqLens.clear();
    kv.currentLen = 0;
    kv.nextFreePage = 0;
}

void kvCacheAppendRope(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, KVCache& kv, const float* newKeys,
                       const float* newValues, uint32_t n, const float* qIn, float* qOut, uint32_t numQHeads,
                       RopeMode mode, float theta, float scaling, int32_t posBase) {
    if (!kv.kPages.valid()) throw std::runtime_error("kvCacheAppend: cache was destroyed");
    if (!newKeys || !newValues) throw std::runtime_error("kvCacheAppend: null tensor pointer");
    if (n == 0) return;
    const auto& c = kv.config;
    grl_device* dev = pool.device().handle();
    if (kv.mla()) {
        // c_t = [k_t | v_t] W_down (kv_cache.cpp:174-248): concatenate, project, store at the current length
        if (mode != RopeMode::None || qIn) throw std::runtime_error("kvCacheAppend: the MLA latent cache takes plain appends (no RoPE, no queries)");
        if (uint32_t(kv.hostSeqLens[0]) + n > kv.capacity())
            throw std::runtime_error("kvCacheAppend: sequence would exceed max_cache_tokens (" + std::to_string(c.maxCacheTokens) + ")");
        cache.getOrCreate("kv-append-mla/" + std::to_string(c.headDim));
        const size_t rows = size_t(n) * c.numHeads, D = c.headDim, L = kv.latentDim;
        GrillyBuffer kb = pool.acquire(rows * D * 4), vb = pool.acquire(rows * D * 4), cat = pool.acquire(rows * 2 * D * 4);
        try {
            Recording rec(batch);
            pool.upload(kb, newKeys, rows * D * 4);
            pool.upload(vb, newValues, rows * D * 4);
            check(grl_mla_concat(dev, static_cast<const float*>(kb.dptr), static_cast<const float*>(vb.dptr),
                                 static_cast<float*>(cat.dptr), rows, int(D)), "kvCacheAppend: concat");
            float* dst = static_cast<float*>(kv.latents.dptr) + size_t(kv.hostSeqLens[0]) * c.numHeads * L;
            check(grl_gemm_f32(dev, static_cast<const float*>(cat.dptr), static_cast<const float*>(kv.wDown.dptr), dst,
                               int(rows), int(2 * D), int(L)), "kvCacheAppend: down-projection");
            kv.hostSeqLens[0] += int32_t(n);
            check(grl_memcpy_h2d(dev, kv.seqLens.dptr, kv.hostSeqLens.data(), 4), "kvCacheAppend: length");
            batch.submit();
        } catch (...) {
            pool.device().quiesce();   // nothing in flight may still touch the buffers released below
            pool.release(kb); pool.release(vb); pool.release(cat);
            throw;
        }
        pool.release(kb); pool.release(vb); pool.release(cat);
        kv.currentLen = uint32_t(kv.hostSeqLens[0]);
        kv.totalAppended += n;
        return;
    }
    cache.getOrCreate("kv-append/" + std::to_string(c.headDim));
    // Overflow: evict what does not fit (lowest cumulative scores, if H2O is on), then compact
    // (kv_cache.cpp:161-172).
    const uint32_t longest = uint32_t(*std::max_element(kv.hostSeqLens.begin(), kv.hostSeqLens.end()));
    if (longest + n > c.maxCacheTokens && longest > 0) {
        if (c.useH2O) kvCacheEvictH2O(batch, pool, cache, kv, nullptr, longest + n - c.maxCacheTokens);
        kvCacheCompact(batch, pool, cache, kv);
    }
    reservePages(pool, kv, n);
    const size_t kvElems = size_t(c.batchSize) * n * c.numHeads * c.headDim;
    const size_t qElems = qIn ? size_t(c.batchSize) * n * numQHeads * c.headDim : 0;
    GrillyBuffer kb = pool.acquire(kvElems * 4), vb = pool.acquire(kvElems * 4), qb, qo;
    if (qIn) { qb = pool.acquire(qElems * 4); qo = pool.acquire(qElems * 4); }
    try {
        Recording rec(batch);
        pool.upload(kb, newKeys, kvElems * 4);
        pool.upload(vb, newValues, kvElems * 4);
        if (qIn) pool.upload(qb, qIn, qElems * 4);
        grl_append_params p{};
        p.kv = kv.layout();
        p.k_new = static_cast<const float*>(kb.dptr);
        p.v_new = static_cast<const float*>(vb.dptr);
        p.q_in = static_cast<const float*>(qb.dptr);
        p.q_out = static_cast<float*>(qo.dptr);
        p.n_new = int(n); p.num_q_heads = int(numQHeads);
        p.rope_mode = int(mode); p.rope_theta = theta; p.rope_scaling = scaling;
        p.pos_base = posBase; p.update_lens = 1;
        p.pos_offsets = static_cast<const int32_t*>(kv.evicted.dptr);
        check(grl_kv_append(dev, &p), "kvCacheAppend");
        if (qIn && qOut) check(grl_memcpy_d2h(dev, qOut, qo.dptr, qElems * 4), "kvCacheAppend: q download");
        batch.submit();
    } catch (...) {
        pool.device().quiesce();   // nothing in flight may still touch the buffers released below
        pool.release(kb); pool.release(vb); pool.release(qb); pool.release(qo);
        throw;
    }
    pool.release(kb); pool.release(vb); pool.release(qb); pool.release(qo);
    for (auto& l : kv.hostSeqLens) l += int32_t(n);
    kv.currentLen = uint32_t(kv.hostSeqLens[0]);
    kv.totalAppended += uint64_t(n) * c.batchSize;
}

void kvCacheAppend(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, KVCache& kv, const float* newKeys,
                   const float* newValues, uint32_t numNewTokens) {
    kvCacheAppendRope(batch, pool, cache, kv, newKeys, newValues, numNewTokens, nullptr, nullptr, 0, RopeMode::None,
                      10000.0f, 1.0f, 0);
}

void kvCacheDecode(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const KVCache& kv, float* decodedKeys,
                   float* decodedValues, uint32_t seq) {
    if (!kv.kPages.valid()) throw std::runtime_error("kvCacheDecode: cache was destroyed");
    const auto& c = kv.config;
    if (seq >= c.batchSize) throw std::runtime_error("kvCacheDecode: sequence index out of range");
    const uint32_t T = uint32_t(kv.hostSeqLens[seq]);
    if (T == 0) return;
    if (!decodedKeys || !decodedValues) throw std::runtime_error("kvCacheDecode: null output");
    grl_device* dev = pool.device().handle();
    if (kv.mla()) {
        // [K | V] = c W_up (kv_cache.cpp:441-498), then split
        cache.getOrCreate("kv-decode-mla/" + std::to_string(c.headDim));
        const size_t rows = size_t(T) * c.numHeads, D = c.headDim, L = kv.latentDim;
        GrillyBuffer full = pool.acquire(rows * 2 * D * 4), kb = pool.acquire(rows * D * 4), vb = pool.acquire(rows * D * 4);
        try {
            Recording rec(batch);
            check(grl_gemm_f32(dev, static_cast<const float*>(kv.latents.dptr), static_cast<const float*>(kv.wUp.dptr),
                               static_cast<float*>(full.dptr), int(rows), int(L), int(2 * D)), "kvCacheDecode: up-projection");
            check(grl_mla_split(dev, static_cast<const float*>(full.dptr), static_cast<float*>(kb.dptr),
                                static_cast<float*>(vb.dptr), rows, int(D)), "kvCacheDecode: split");
            check(grl_memcpy_d2h(dev, decodedKeys, kb.dptr, rows * D * 4), "kvCacheDecode: download");
            check(grl_memcpy_d2h(dev, decodedValues, vb.dptr, rows * D * 4), "kvCacheDecode: download");
            batch.submit();
        } catch (...) {
            pool.device().quiesce();   // nothing in flight may still touch the buffers released below
            pool.release(full); pool.release(kb); pool.release(vb);
            throw;
        }
        pool.release(full); pool.release(kb); pool.release(vb);
        return;
    }
    cache.getOrCreate("kv-gather/" + std::to_string(c.headDim));
    const size_t n = size_t(T) * c.numHeads * c.headDim;
    GrillyBuffer kb = pool.acquire(n * 4), vb = pool.acquire(n * 4);
    try {
        Recording rec(batch);
        grl_kv_layout l = kv.layout();
        check(grl_kv_gather(dev, &l, int(seq), int(T), static_cast<float*>(kb.dptr), static_cast<float*>(vb.dptr)),
              "kvCacheDecode");
        check(grl_memcpy_d2h(dev, decodedKeys, kb.dptr, n * 4), "kvCacheDecode: download");
        check(grl_memcpy_d2h(dev, decodedValues, vb.dptr, n * 4), "kvCacheDecode: download");
        batch.submit();
    } catch (...) {
        pool.device().quiesce();   // nothing in flight may still touch the buffers released below
        pool.release(kb); pool.release(vb);
        throw;
    }
    pool.release(kb); pool.release(vb);
}

void kvCacheSetMLAWeights(BufferPool& pool, KVCache& kv, const float* wDown, const float* wUp) {
    if (!kv.mla()) throw std::runtime_error("kvCacheSetMLAWeights: not an MLA cache (compression_ratio > 1)");
    if (!wDown || !wUp) throw std::runtime_error("kvCacheSetMLAWeights: null matrix");
    grl_device* dev = pool.device().handle();
    const size_t bytes = size_t(2) * kv.config.headDim * kv.latentDim * 4;
    check(grl_memcpy_h2d(dev, kv.wDown.dptr, wDown, bytes), "kvCacheSetMLAWeights");
    check(grl_memcpy_h2d(dev, kv.wUp.dptr, wUp, bytes), "kvCacheSetMLAWeights");
    check(grl_sync(dev, 0), "kvCacheSetMLAWeights");
}

KVCacheStats kvCacheGetStats(const KVCache& kv) {
    KVCacheStats s{};
    s.currentTokens = kv.currentLen;
    s.maxTokens = kv.config.maxCacheTokens;
    s.totalEvicted = uint32_t(kv.totalEvicted);
    s.totalAppended = uint32_t(kv.totalAppended);
    // bytes saved against float32 storage
    s.compressionRatio = kv.config.dtype == GRL_BF16 ? 2.0f : kv.config.dtype == GRL_FP8_INT4 ? 8.0f / 1.5f : 1.0f;   // the scales are not counted (kv_cache.cpp:1024-1027)
    if (kv.mla()) s.compressionRatio = 2.0f * float(kv.config.headDim) / float(kv.latentDim);   // kv_cache.cpp:1017-1020
    // mean cumulative score of the active tokens of sequence 0, summed in index order (kv_cache.cpp:1004-1015)
    s.avgAttentionScore = 0.0f;
    if (kv.device && kv.cumScore.valid() && kv.currentLen > 0) {
        std::vector<float> cum(kv.currentLen);
        std::vector<uint8_t> tomb(kv.currentLen);
        check(grl_memcpy_d2h(kv.device, cum.data(), kv.cumScore.dptr, cum.size() * 4), "kvCacheGetStats");
        check(grl_memcpy_d2h(kv.device, tomb.data(), kv.tombstone.dptr, tomb.size()), "kvCacheGetStats");
        check(grl_sync(kv.device, 0), "kvCacheGetStats");
        float total = 0.0f;
        uint32_t active = 0;
        for (uint32_t t = 0; t < kv.currentLen; ++t)
            if (!tomb[t]) { total += cum[t]; ++active; }
        if (active) s.avgAttentionScore = total / float(active);
    }
    s.pagesTotal = kv.numPages;
    s.pagesUsed = kv.nextFreePage;
    s.bytes = uint64_t(kv.kPages.bucketSize) + kv.vPages.bucketSize + kv.scales.bucketSize;
    return s;
}

// Queues the decode of q over the cache.  With `track`, the step also adds the attention mass every cached
// token received (summed over the query heads) to the cache's cumulative scores -- what H2O eviction
// ranks by: the kernel leaves its scaled scores and an un-normalised result, a merge of one part
// normalises it, and grl_kv_mass_accumulate turns scores into probabilities.
static void launchDecode(grl_device* dev, BufferPool& pool, const KVCache& kv, const float* qDev, float* outDev,
                         uint32_t numQHeads, float scale, int nSplits, GrillyBuffer& ws, bool track = false) {
    grl_decode_params p{};
    p.kv = kv.layout();
    p.q = qDev; p.out = outDev;
    p.num_q_heads = int(numQHeads);
    p.scale = scale; p.n_splits = nSplits;
    p.max_seq_len = *std::max_element(kv.hostSeqLens.begin(), kv.hostSeqLens.end());
    int splits = 0;
    check(grl_decode_pick_splits(dev, &p, &splits), "gqaAttention");
    size_t bytes = 0;
    check(grl_decode_workspace_bytes(&p, splits, &bytes), "gqaAttention");
    const size_t rows = size_t(kv.config.batchSize) * numQHeads, D = kv.config.headDim;
    const size_t ld = (size_t(p.max_seq_len) + 3) / 4 * 4;
    const size_t partBytes = rows * (D + 2) * 4, scoreBytes = rows * ld * 4;
    const size_t wsBytes = (bytes + 255) / 256 * 256;
    ws = pool.acquire(wsBytes + (track ? partBytes + 256 + scoreBytes : 0));
    p.n_splits = splits; p.workspace = ws.dptr; p.workspace_bytes = wsBytes;
    if (!track) {
        check(grl_gqa_decode(dev, &p), "gqaAttention");
        return;
    }
    float* part = reinterpret_cast<float*>(static_cast<char*>(ws.dptr) + wsBytes);
    float* scores = reinterpret_cast<float*>(static_cast<char*>(ws.dptr) + wsBytes + (partBytes + 255) / 256 * 256);
    p.out = nullptr; p.partial_out = part;
    p.scores_out = scores; p.scores_ld = int(ld);
    check(grl_gqa_decode(dev, &p), "gqaAttention");
    check(grl_lse_merge(dev, part, 1, rows * (D + 2), int(rows), int(D), 1, outDev), "gqaAttention: normalise");
    grl_kv_meta m = kv.meta();
    check(grl_kv_mass_accumulate(dev, &p.kv, &m, scores, int(ld), part, int(numQHeads)), "gqaAttention: scores");
}

void gqaAttention(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const KVCache& kv, const float* q,
                  float* out, uint32_t numQHeads, float scale, int nSplits, bool accumulateScores) {
    if (!kv.kPages.valid()) throw std::runtime_error("gqaAttention: cache was destroyed");
    if (kv.mla()) throw std::runtime_error("gqaAttention: not built for the MLA latent cache (decode it with kvCacheDecode, or use compression_ratio=1)");
    if (!q || !out) throw std::runtime_error("gqaAttention: null tensor pointer");
    const auto& c = kv.config;
    if (numQHeads == 0 || numQHeads % c.numHeads != 0)
        throw std::runtime_error("gqaAttention: num_q_heads must be a positive multiple of num_kv_heads");
    grl_device* dev = pool.device().handle();
    cache.getOrCreate("gqa-attention/" + std::to_string(c.headDim));
    const size_t n = size_t(c.batchSize) * numQHeads * c.headDim;
    GrillyBuffer qb = pool.acquire(n * 4), ob = pool.acquire(n * 4), ws;
    try {
        Recording rec(batch);
        pool.upload(qb, q, n * 4);
        launchDecode(dev, pool, kv, static_cast<const float*>(qb.dptr), static_cast<float*>(ob.dptr), numQHeads, scale,
                     nSplits, ws, accumulateScores);
        check(grl_memcpy_d2h(dev, out, ob.dptr, n * 4), "gqaAttention: download");
        batch.submit();
    } catch (...) {
        pool.device().quiesce();   // nothing in flight may still touch the buffers released below
        pool.release(qb); pool.release(ob); pool.release(ws);
        throw;
    }
    pool.release(qb); pool.release(ob); pool.release(ws);
}

void decodeStep(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, KVCache& kv, const float* q,
                const float* kNew, const float* vNew, float* out, uint32_t numQHeads, RopeMode mode, float theta,
                float scaling, float scale, bool accumulateScores) {
    if (!kv.kPages.valid()) throw std::runtime_error("decodeStep: cache was destroyed");
    if (kv.mla()) throw std::runtime_error("decodeStep: not built for the MLA latent cache (decode it with kvCacheDecode, or use compression_ratio=1)");
    if (!q || !kNew || !vNew || !out) throw std::runtime_error("decodeStep: null tensor pointer");
    const auto& c = kv.config;
    if (numQHeads == 0 || numQHeads % c.numHeads != 0)
        throw std::runtime_error("decodeStep: num_q_heads must be a positive multiple of num_kv_heads");
    grl_device* dev = pool.device().handle();
    cache.getOrCreate("decode-step/" + std::to_string(c.headDim));
    reservePages(pool, kv, 1);
    const size_t qn = size_t(c.batchSize) * numQHeads * c.headDim, kn = size_t(c.batchSize) * c.numHeads * c.headDim;
    GrillyBuffer qb = pool.acquire(qn * 4), qr = pool.acquire(qn * 4), ob = pool.acquire(qn * 4),
                 kb = pool.acquire(kn * 4), vb = pool.acquire(kn * 4), ws;
    auto releaseAll = [&]() {
        pool.release(qb); pool.release(qr); pool.release(ob); pool.release(kb); pool.release(vb); pool.release(ws);
    };
    try {
        Recording rec(batch);
        pool.upload(qb, q, qn * 4);
        pool.upload(kb, kNew, kn * 4);
        pool.upload(vb, vNew, kn * 4);
        grl_append_params ap{};
        ap.kv = kv.layout();
        ap.k_new = static_cast<const float*>(kb.dptr);
        ap.v_new = static_cast<const float*>(vb.dptr);
        ap.q_in = static_cast<const float*>(qb.dptr);
        ap.q_out = static_cast<float*>(qr.dptr);
        ap.n_new = 1; ap.num_q_heads = int(numQHeads);
        ap.rope_mode = int(mode); ap.rope_theta = theta; ap.rope_scaling = scaling;
        ap.pos_base = 0; ap.update_lens = 1;
        ap.pos_offsets = static_cast<const int32_t*>(kv.evicted.dptr);
        check(grl_kv_append(dev, &ap), "decodeStep: append");
        for (auto& l : kv.hostSeqLens) l += 1;
        kv.currentLen = uint32_t(kv.hostSeqLens[0]);
        kv.totalAppended += c.batchSize;
        launchDecode(dev, pool, kv, static_cast<const float*>(qr.dptr), static_cast<float*>(ob.dptr), numQHeads, scale,
                     0, ws, accumulateScores);
        check(grl_memcpy_d2h(dev, out, ob.dptr, qn * 4), "decodeStep: download");
        batch.submit();
    } catch (...) {
        pool.device().quiesce();   // nothing in flight may still touch the buffers released below
        releaseAll();
        throw;
    }
    releaseAll();
}

void gqaAttentionDevice(BufferPool& pool, PipelineCache& cache, const KVCache& kv, const GrillyBuffer& q,
                        GrillyBuffer& out, uint32_t numQHeads, float scale, int nSplits, GrillyBuffer& ws) {
    if (!kv.kPages.valid()) throw std::runtime_error("gqaAttention: cache was destroyed");
    if (kv.mla()) throw std::runtime_error("gqaAttention: not built for the MLA latent cache (decode it with kvCacheDecode, or use compression_ratio=1)");
    const auto& c = kv.config;
    if (numQHeads == 0 || numQHeads % c.numHeads != 0)
        throw std::runtime_error("gqaAttention: num_q_heads must be a positive multiple of num_kv_heads");
    const size_t bytes = size_t(c.batchSize) * numQHeads * c.headDim * 4;
    if (q.size < bytes || out.size < bytes) throw std::runtime_error("gqaAttention: q / out buffer too small");
    cache.getOrCreate("gqa-attention-device/" + std::to_string(c.headDim));
    launchDecode(pool.device().handle(), pool, kv, static_cast<const float*>(q.dptr), static_cast<float*>(out.dptr),
                 numQHeads, scale, nSplits, ws);
}

void decodeStepDevice(BufferPool& pool, PipelineCache& cache, KVCache& kv, const GrillyBuffer& q,
                      const GrillyBuffer& kNew, const GrillyBuffer& vNew, GrillyBuffer& qRotated, GrillyBuffer& out,
                      uint32_t numQHeads, RopeMode mode, float theta, float scaling, float scale, GrillyBuffer& ws) {
    if (!kv.kPages.valid()) throw std::runtime_error("decodeStep: cache was destroyed");
    if (kv.mla()) throw std::runtime_error("decodeStep: not built for the MLA latent cache (decode it with kvCacheDecode, or use compression_ratio=1)");
    const auto& c = kv.config;
    if (numQHeads == 0 || numQHeads % c.numHeads != 0)
        throw std::runtime_error("decodeStep: num_q_heads must be a positive multiple of num_kv_heads");
    const size_t qb = size_t(c.batchSize) * numQHeads * c.headDim * 4, kb = size_t(c.batchSize) * c.numHeads * c.headDim * 4;
    if (q.size < qb || qRotated.size < qb || out.size < qb || kNew.size < kb || vNew.size < kb)
        throw std::runtime_error("decodeStep: buffer too small");
    grl_device* dev = pool.device().handle();
    cache.getOrCreate("decode-step-device/" + std::to_string(c.headDim));
    reservePages(pool, kv, 1);
    grl_append_params ap{};
    ap.kv = kv.layout();
    ap.k_new = static_cast<const float*>(kNew.dptr);
    ap.v_new = static_cast<const float*>(vNew.dptr);
    ap.q_in = static_cast<const float*>(q.dptr);
    ap.q_out = static_cast<float*>(qRotated.dptr);
    ap.n_new = 1; ap.num_q_heads = int(numQHeads);
    ap.rope_mode = int(mode); ap.rope_theta = theta; ap.rope_scaling = scaling;
    ap.pos_base = 0; ap.update_lens = 1;
    ap.pos_offsets = static_cast<const int32_t*>(kv.evicted.dptr);
    check(grl_kv_append(dev, &ap), "decodeStep: append");
    for (auto& l : kv.hostSeqLens) l += 1;
    kv.currentLen = uint32_t(kv.hostSeqLens[0]);
    kv.totalAppended += c.batchSize;
    launchDecode(dev, pool, kv, static_cast<const float*>(qRotated.dptr), static_cast<float*>(out.dptr), numQHeads, scale, 0, ws);
}

void kvCacheEvictH2O(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, KVCache& kv,
                     const float* attentionScores, uint32_t numEvict) {
    if (!kv.kPages.valid()) throw std::runtime_error("kvCacheEvictH2O: cache was destroyed");
    const auto& c = kv.config;
    // nothing to do where the count reaches the length -- decided before the scores are touched, as the
    // reference does (kv_cache.cpp:598-601); with ragged sequences the kernels apply it per sequence
    bool any = false;
    for (int32_t len : kv.hostSeqLens) {
        const uint32_t k = numEvict ? numEvict : uint32_t(len) / 4;
        if (k < uint32_t(len)) any = true;
    }
    if (!any) return;
    grl_device* dev = pool.device().handle();
    cache.getOrCreate("kv-evict-h2o");
    grl_kv_layout l = kv.layout();
    grl_kv_meta m = kv.meta();
    GrillyBuffer scores;
    try {
        Recording rec(batch);
        if (attentionScores) {
            const uint32_t T = uint32_t(kv.hostSeqLens[0]);
            for (int32_t len : kv.hostSeqLens)
                if (uint32_t(len) != T)
                    throw std::runtime_error("kvCacheEvictH2O: attention scores need sequences of equal length");
            const size_t n = size_t(c.batchSize) * T * T;
            scores = pool.acquire(n * 4);
            pool.upload(scores, attentionScores, n * 4);
            check(grl_kv_score_accumulate(dev, &l, &m, static_cast<const float*>(scores.dptr), int(T), int(T)),
                  "kvCacheEvictH2O: accumulate");
        }
        check(grl_kv_evict_lowest(dev, &l, &m, int(numEvict)), "kvCacheEvictH2O");
        batch.submit();
    } catch (...) {
        pool.device().quiesce();   // nothing in flight may still touch the buffers released below
        pool.release(scores);
        throw;
    }
    pool.release(scores);
}

void kvCacheInitEvictionHead(BufferPool& pool, KVCache& kv, uint32_t inputDim, uint32_t hiddenDim, float lr) {
    if (!kv.kPages.valid()) throw std::runtime_error("kvCacheInitEvictionHead: cache was destroyed");
    if (kv.config.batchSize != 1) throw std::runtime_error("kvCacheInitEvictionHead: single-sequence caches only");
    if (inputDim == 0 || hiddenDim == 0) throw std::runtime_error("kvCacheInitEvictionHead: empty shape");
    kvCacheDestroyEvictionHead(pool, kv);
    auto& head = kv.evictionHead;
    head.inputDim = inputDim; head.hiddenDim = hiddenDim; head.learningRate = lr; head.totalUpdates = 0;
    head.w1 = pool.acquire(size_t(inputDim) * hiddenDim * 4);
    head.b1 = pool.acquire(size_t(hiddenDim) * 4);
    head.w2 = pool.acquire(size_t(hiddenDim) * 4);
    head.b2 = pool.acquire(4);
    // Xavier-uniform from rand(), W1 first then W2, biases zero -- the draw order of kv_cache.cpp:676-701
    const float x1 = std::sqrt(6.0f / float(inputDim + hiddenDim));
    std::vector<float> w1(size_t(inputDim) * hiddenDim);
    for (auto& v : w1) v = (static_cast<float>(rand()) / RAND_MAX * 2.0f - 1.0f) * x1;
    const float x2 = std::sqrt(6.0f / float(hiddenDim + 1));
    std::vector<float> w2(hiddenDim);
    for (auto& v : w2) v = (static_cast<float>(rand()) / RAND_MAX * 2.0f - 1.0f) * x2;
    grl_device* dev = pool.device().handle();
    check(grl_memcpy_h2d(dev, head.w1.dptr, w1.data(), w1.size() * 4), "kvCacheInitEvictionHead");
    check(grl_memcpy_h2d(dev, head.w2.dptr, w2.data(), w2.size() * 4), "kvCacheInitEvictionHead");
    check(grl_memset(dev, head.b1.dptr, 0, size_t(hiddenDim) * 4), "kvCacheInitEvictionHead");
    check(grl_memset(dev, head.b2.dptr, 0, 4), "kvCacheInitEvictionHead");
    check(grl_sync(dev, 0), "kvCacheInitEvictionHead");
    head.initialized = true;
}

void kvCacheDestroyEvictionHead(BufferPool& pool, KVCache& kv) {
    auto& head = kv.evictionHead;
    if (!head.initialized) return;
    pool.release(head.w1); pool.release(head.b1); pool.release(head.w2); pool.release(head.b2);
    head.initialized = false;
}

void kvCacheTrainEvictionHead(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, KVCache& kv,
                              const float* tokenFeatures, const float* attentionScores, uint32_t seqLen) {
    auto& head = kv.evictionHead;
    if (!head.initialized) return;                    // kv_cache.cpp:741
    const uint32_t T = kv.currentLen;
    if (T == 0) return;
    if (!tokenFeatures || !attentionScores || seqLen == 0)
        throw std::runtime_error("kvCacheTrainEvictionHead: null features / scores");
    grl_device* dev = pool.device().handle();
    cache.getOrCreate("kv-eviction-head-train");
    grl_kv_layout l = kv.layout();
    grl_kv_meta m = kv.meta();
    grl_evict_head hv = head.view();
    size_t bytes = 0;
    check(grl_evict_head_scratch_bytes(&hv, int(T), &bytes), "kvCacheTrainEvictionHead");
    GrillyBuffer feat = pool.acquire(size_t(T) * head.inputDim * 4), attn = pool.acquire(size_t(seqLen) * T * 4),
                 scratch = pool.acquire(bytes);
    try {
        Recording rec(batch);
        pool.upload(feat, tokenFeatures, size_t(T) * head.inputDim * 4);
        pool.upload(attn, attentionScores, size_t(seqLen) * T * 4);
        check(grl_evict_head_train(dev, &l, &m, &hv, static_cast<const float*>(feat.dptr),
                                   static_cast<const float*>(attn.dptr), int(seqLen), int(T), head.learningRate,
                                   scratch.dptr, scratch.bucketSize),
              "kvCacheTrainEvictionHead");
        batch.submit();
    } catch (...) {
        pool.device().quiesce();   // nothing in flight may still touch the buffers released below
        pool.release(feat); pool.release(attn); pool.release(scratch);
        throw;
    }
    pool.release(feat); pool.release(attn); pool.release(scratch);
    head.totalUpdates++;
}

void kvCacheEvictSpeculative(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, KVCache& kv,
                             const float* hiddenStates, uint32_t /*hiddenDim: the reference strides by head.inputDim*/) {
    if (!kv.kPages.valid()) throw std::runtime_error("kvCacheEvictSpeculative: cache was destroyed");
    grl_device* dev = pool.device().handle();
    grl_kv_layout l = kv.layout();
    grl_kv_meta m = kv.meta();
    const auto& head = kv.evictionHead;
    if (head.initialized && head.totalUpdates > 0 && hiddenStates && kv.currentLen > 0) {   // kv_cache.cpp:863-866
        cache.getOrCreate("kv-eviction-head-predict");
        grl_evict_head hv = head.view();
        const size_t n = size_t(kv.currentLen) * head.inputDim;
        GrillyBuffer feat = pool.acquire(n * 4);
        try {
            Recording rec(batch);
            pool.upload(feat, hiddenStates, n * 4);
            check(grl_evict_head_predict(dev, &l, &m, &hv, static_cast<const float*>(feat.dptr), int(kv.currentLen),
                                         kv.config.evictionThreshold),
                  "kvCacheEvictSpeculative");
            batch.submit();
        } catch (...) {
            pool.device().quiesce();   // nothing in flight may still touch the buffers released below
            pool.release(feat);
            throw;
        }
        pool.release(feat);
        return;
    }
    cache.getOrCreate("kv-evict-heuristic");
    Recording rec(batch);
    check(grl_kv_evict_heuristic(dev, &l, &m, kv.config.evictionThreshold), "kvCacheEvictSpeculative");
    batch.submit();
}

void kvCacheCompact(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, KVCache& kv) {
    if (!kv.kPages.valid()) throw std::runtime_error("kvCacheCompact: cache was destroyed");
    if (kv.mla()) throw std::runtime_error("kvCacheCompact: not built for the MLA latent cache (decode it with kvCacheDecode, or use compression_ratio=1)");
    grl_device* dev = pool.device().handle();
    cache.getOrCreate("kv-compact/" + std::to_string(kv.config.headDim));
    grl_kv_layout l = kv.layout();
    grl_kv_meta m = kv.meta();
    size_t bytes = 0;
    check(grl_kv_compact_scratch_bytes(&l, &m, &bytes), "kvCacheCompact");
    GrillyBuffer scratch = pool.acquire(bytes);
    std::vector<int32_t> lens(kv.config.batchSize);
    try {
        Recording rec(batch);
        check(grl_kv_compact(dev, &l, &m, scratch.dptr, scratch.bucketSize), "kvCacheCompact");
        check(grl_memcpy_d2h(dev, lens.data(), kv.seqLens.dptr, lens.size() * 4), "kvCacheCompact: lengths");
        batch.submit();
    } catch (...) {
        pool.device().quiesce();   // nothing in flight may still touch the buffers released below
        pool.release(scratch);
        throw;
    }
    pool.release(scratch);
    for (size_t b = 0; b < lens.size(); ++b) {
        kv.totalEvicted += uint64_t(kv.hostSeqLens[b] - lens[b]);
        kv.hostSeqLens[b] = lens[b];
    }
    kv.currentLen = uint32_t(kv.hostSeqLens[0]);
}

void kvCacheTokenMeta(BufferPool& pool, const KVCache& kv, uint32_t seq, std::vector<float>& cumScore,
                      std::vector<uint8_t>& tombstone, std::vector<float>& relevance) {
    if (!kv.kPages.valid()) throw std::runtime_error("kvCacheTokenMeta: cache was destroyed");
    if (seq >= kv.config.batchSize) throw std::runtime_error("kvCacheTokenMeta: sequence index out of range");
    const size_t T = size_t(kv.hostSeqLens[seq]), off = size_t(seq) * kv.capacity();
    cumScore.resize(T); tombstone.resize(T); relevance.resize(T);
    if (T == 0) return;
    grl_device* dev = pool.device().handle();
    check(grl_memcpy_d2h(dev, cumScore.data(), static_cast<const float*>(kv.cumScore.dptr) + off, T * 4), "kvCacheTokenMeta");
    check(grl_memcpy_d2h(dev, tombstone.data(), static_cast<const uint8_t*>(kv.tombstone.dptr) + off, T), "kvCacheTokenMeta");
    check(grl_memcpy_d2h(dev, relevance.data(), static_cast<const float*>(kv.relevance.dptr) + off, T * 4), "kvCacheTokenMeta");
    check(grl_sync(dev, 0), "kvCacheTokenMeta");
}

}  // namespace ops
}  // namespace grilly

// KV-sharded decode across GPUs: local split-KV decode -> NCCL all-gather of partials -> LSE merge.
#include <algorithm>
#include <stdexcept>
#include <string>

#include "grilly/ops/sharded_decode.h"

namespace grilly {
namespace ops {

std::array<uint8_t, 128> shardGroupUniqueId() {
    std::array<uint8_t, 128> id{};
    check(grl_group_unique_id(id.data()), "shardGroupUniqueId");
    return id;
}

ShardGroup createShardGroup(GrillyDevice& device, const uint8_t* id128, int rank, int world) {
    if (!id128) throw std::runtime_error("createShardGroup: id is null");
    ShardGroup g;
    g.rank = rank;
    g.world = world;
    check(grl_group_init_rank(device.handle(), id128, rank, world, &g.group), "createShardGroup");
    return g;
}

void destroyShardGroup(BufferPool& pool, ShardGroup& g) {
    if (g.group) {
        grl_group_destroy(g.group);
        g.group = nullptr;
    }
    pool.release(g.partial);
    pool.release(g.gathered);
}

std::pair<uint64_t, uint64_t> shardRange(uint64_t totalTokens, int world, int rank) {
    if (world <= 0 || rank < 0 || rank >= world) throw std::runtime_error("shardRange: bad rank / world");
    const uint64_t base = totalTokens / uint64_t(world), rem = totalTokens % uint64_t(world);
    const uint64_t start = uint64_t(rank) * base + std::min<uint64_t>(uint64_t(rank), rem);
    return {start, start + base + (uint64_t(rank) < rem ? 1 : 0)};
}

void shardedDecodeStep(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const KVCache& kv, ShardGroup& g,
                       const float* q, float* out, uint32_t numQHeads, float scale, uint64_t timeoutNs) {
    if (!g.group) throw std::runtime_error("shardedDecodeStep: the group was destroyed");
    if (!kv.kPages.valid()) throw std::runtime_error("shardedDecodeStep: cache was destroyed");
    if (kv.mla()) throw std::runtime_error("shardedDecodeStep: not built for the MLA latent cache");
    if (!q || !out) throw std::runtime_error("shardedDecodeStep: null tensor pointer");
    const auto& c = kv.config;
    if (numQHeads == 0 || numQHeads % c.numHeads != 0)
        throw std::runtime_error("shardedDecodeStep: num_q_heads must be a positive multiple of num_kv_heads");
    grl_device* dev = pool.device().handle();
    cache.getOrCreate("sharded-decode/" + std::to_string(c.headDim));
    const size_t rows = size_t(c.batchSize) * numQHeads, D = c.headDim;
    const size_t n = rows * D, partFloats = rows * (D + 2);
    if (g.partial.size < partFloats * 4) {
        pool.release(g.partial);
        pool.release(g.gathered);
        g.partial = pool.acquire(partFloats * 4);
        g.gathered = pool.acquire(partFloats * 4 * size_t(g.world));
    }
    GrillyBuffer qb = pool.acquire(n * 4), ob = pool.acquire(n * 4), ws;
    auto releaseAll = [&]() { pool.release(qb); pool.release(ob); pool.release(ws); };
    try {
        batch.begin();
        pool.upload(qb, q, n * 4);
        grl_decode_params p{};
        p.kv = kv.layout();
        p.q = static_cast<const float*>(qb.dptr);
        p.num_q_heads = int(numQHeads);
        p.scale = scale;
        p.max_seq_len = std::max(1, *std::max_element(kv.hostSeqLens.begin(), kv.hostSeqLens.end()));
        int splits = 0;
        check(grl_decode_pick_splits(dev, &p, &splits), "shardedDecodeStep");
        size_t bytes = 0;
        check(grl_decode_workspace_bytes(&p, splits, &bytes), "shardedDecodeStep");
        ws = pool.acquire(std::max<size_t>(bytes, 256));
        p.n_splits = splits; p.workspace = ws.dptr; p.workspace_bytes = ws.bucketSize;
        p.partial_out = static_cast<float*>(g.partial.dptr);     // an empty shard leaves (0, -1e30, 0): weight zero
        check(grl_gqa_decode(dev, &p), "shardedDecodeStep: decode");
        check(grl_group_allgather_merge(g.group, static_cast<const float*>(g.partial.dptr), int(rows), int(D),
                                        static_cast<float*>(g.gathered.dptr), static_cast<float*>(ob.dptr), 0),
              "shardedDecodeStep: all-gather + merge");
        check(grl_memcpy_d2h(dev, out, ob.dptr, n * 4), "shardedDecodeStep: download");
        batch.submitNoWait();
        check(grl_group_sync(g.group, timeoutNs), "shardedDecodeStep");
    } catch (...) {
        if (batch.recording()) batch.submitNoWait();
        pool.device().quiesce();   // nothing in flight may still touch the buffers released below
        releaseAll();
        throw;
    }
    releaseAll();
}

}  // namespace ops
}  // namespace grilly

#pragma once
// Long-context decode with the KV sequence sharded over GPUs, one process per GPU.
//
// The reference has no multi-GPU code; this op extends its decode step
// (shaders/gqa-attention.glsl:34-130) across devices: rank g of G holds a contiguous range of every
// sequence's tokens in its own paged KVCache; a step is the split-KV decode over the local shard to one
// un-normalised partial [O | m | l], an all-gather of the partials over NVLink (NCCL, behind the C ABI's
// grl_group_*), and the log-sum-exp merge on every rank.
#include <array>
#include <cstdint>

#include "grilly/ops/kv_cache.h"

namespace grilly {
namespace ops {

struct ShardGroup {
    grl_group* group = nullptr;
    int rank = 0, world = 1;
    GrillyBuffer partial, gathered;   // [rows*(D+2)] and world times that, float32 in HBM
};

/// Rank 0 makes the id and hands it to the other ranks over any host channel (a socket, a file, MPI ...).
std::array<uint8_t, 128> shardGroupUniqueId();
/// Collective: every rank of the group calls it with the same id.
ShardGroup createShardGroup(GrillyDevice& device, const uint8_t* id128, int rank, int world);
void destroyShardGroup(BufferPool& pool, ShardGroup& group);

/// Token range [first, second) of `rank` when `totalTokens` are split into `world` contiguous shards.
std::pair<uint64_t, uint64_t> shardRange(uint64_t totalTokens, int world, int rank);

/// One decode step.  kvCache holds this rank's token range; q (B,1,Hq,D) host float32, already rotated and
/// identical on every rank; out (B,1,Hq,D) receives the attention over ALL ranks' tokens.  Synchronous;
/// throws std::runtime_error when the collective fails or does not finish within timeoutNs (the group is
/// then aborted and only good for destroyShardGroup).
void shardedDecodeStep(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const KVCache& kvCache,
                       ShardGroup& group, const float* q, float* out, uint32_t numQHeads, float scale = 0.0f,
                       uint64_t timeoutNs = 2000000000ull);

}  // namespace ops
}  // namespace grilly

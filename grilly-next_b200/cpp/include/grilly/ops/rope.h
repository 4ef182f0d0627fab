#pragma once
// Standalone RoPE and attention-mask ops with the push-constant contracts of
// shaders/rope.glsl:32-40 and shaders/attention-mask.glsl:18-24 (the reference ships the shaders
// without a C++ dispatcher; these follow its op-layer conventions).
#include <cstdint>

#include "grilly/buffer_pool.h"
#include "grilly/command_batch.h"
#include "grilly/ops/attention.h"
#include "grilly/pipeline_cache.h"

namespace grilly {
namespace ops {

/// x, y: (B,S,H,D) float32 host arrays.  cosTable/sinTable: nullptr or (>=S, D/2) float32.
void rope(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* x, float* y, uint32_t batchSize,
          uint32_t seqLen, uint32_t numHeads, uint32_t headDim, float base = 10000.0f, float scaling = 1.0f,
          RopeMode mode = RopeMode::Half, const float* cosTable = nullptr, const float* sinTable = nullptr);

/// scores: (B,H,S,S) float32 host array, modified in place.  keyMask: (B,S) or nullptr with causal.
void attentionMask(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, float* scores, const float* keyMask,
                   uint32_t batchSize, uint32_t numHeads, uint32_t seqLen, bool causal, float maskValue = -1e9f);

}  // namespace ops
}  // namespace grilly

#pragma once
// Prefill attention ops.  flashAttention2 keeps the reference signature
// (cpp/include/grilly/ops/attention.h:55-62); flashAttention2Ex adds the implicit masks, RoPE
// and the bf16 tensor-core path; the *Device forms take HBM-resident buffers.
#include <cstdint>

#include "grilly/buffer_pool.h"
#include "grilly/command_batch.h"
#include "grilly/pipeline_cache.h"

namespace grilly {
namespace ops {

/// Push-constant block of the reference shader (flash-attention2.glsl:49-61), kept as a public POD.
struct FlashAttention2Params {
    uint32_t batchSize, seqLen, numHeads, headDim;
    float scale;
    uint32_t tileSizeQ, tileSizeK, passType, hasMask, qTileIdx, kTileIdx;
};

enum class RopeMode : int { None = GRL_ROPE_NONE, Interleaved = GRL_ROPE_INTERLEAVED, Half = GRL_ROPE_HALF };
enum class Precision : int { FP32 = 0, BF16 = 1 };

/// Extensions over the reference call: everything defaults to the reference behaviour.
struct FlashAttention2Options {
    bool causal = false;
    const int32_t* seqLens = nullptr;   // host, (batch) valid lengths; rows beyond are zero
    int maskRank = 4;                   // rank of `mask`: 2 (B,S), 3 (B,S,S), 4 (B,H,S,S)
    bool maskBroadcastHeads = false;    // rank 4 with a head extent of 1
    RopeMode ropeMode = RopeMode::None;
    float ropeTheta = 10000.0f;         // rope_base of flash-attention2-rope.glsl:56-71
    float ropeScaling = 1.0f;
    Precision precision = Precision::FP32;  // BF16: inputs rounded to bf16, tcgen05 kernel
};

/// What the last chunked (pipelined) flashAttention2 call of this process did: the share of every chunk that
/// the host threads rounded to bf16 themselves, and the busy time of each stage -- host rounding (wall clock of
/// the calling thread), upload queue, main queue (device cast + attention kernel), download queue (CUDA events,
/// summed over the chunks) -- against the wall time of the whole call.  The stages overlap; the longest one
/// names the limiter.  Queue times are collected only while setPipelineTiming(true) is in force.
struct PipelineInfo {
    bool valid = false, timed = false;
    int hostCastPct = 0, chunks = 0, hostThreads = 0;
    double hostRoundMs = 0, h2dMs = 0, kernelMs = 0, d2hMs = 0, totalMs = 0;
    double h2dBytes = 0, d2hBytes = 0, hostRoundBytes = 0;
};
PipelineInfo lastPipelineInfo();
void setPipelineTiming(bool on);

/// Host pointers in, host pointer out, synchronous -- the reference contract
/// (cpp/src/ops/attention.cpp:45-166).  Q,K,V,output: (B,H,S,D) float32 row-major;
/// mask: nullptr or (B,H,S,S) floats, > 0 keeps.
void flashAttention2(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* Q, const float* K,
                     const float* V, const float* mask, float* output, uint32_t batchSize, uint32_t seqLen,
                     uint32_t numHeads, uint32_t headDim, float scale = 0.0f, uint32_t tileSizeQ = 64,
                     uint32_t tileSizeK = 64);

void flashAttention2Ex(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* Q, const float* K,
                       const float* V, const float* mask, float* output, uint32_t batchSize, uint32_t seqLen,
                       uint32_t numHeads, uint32_t headDim, float scale, const FlashAttention2Options& opt);

/// Device-resident form: q,k,v,out are HBM buffers of dtype inDtype/outDtype (GRL_F32 / GRL_BF16),
/// seqLensDev a device int32 buffer or empty.  Asynchronous on the context stream.
void flashAttention2Device(CommandBatch& batch, PipelineCache& cache, const GrillyBuffer& q, const GrillyBuffer& k,
                           const GrillyBuffer& v, GrillyBuffer& out, int inDtype, int outDtype, uint32_t batchSize,
                           uint32_t seqLen, uint32_t numHeads, uint32_t headDim, float scale, bool causal,
                           const GrillyBuffer* seqLensDev, RopeMode ropeMode, float ropeTheta, float ropeScaling);

/// Bytes of the swizzled form of a (B,H,S,D) float32 tensor (cpp/src/ops/swizzle.cpp swizzledBufferSize).
size_t swizzledBufferSize(uint32_t batchSize, uint32_t numHeads, uint32_t seqLen, uint32_t headDim, uint32_t waveSize = 32);
/// (B,H,S,D) -> (B,H,S_pad/W,D_pad/W,W,W) with zero padding, or back with reverse: host pointers, synchronous
/// (the reference's ops::swizzle, cpp/src/ops/swizzle.cpp:164-229).
void swizzle(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* input, float* output,
             uint32_t batchSize, uint32_t numHeads, uint32_t seqLen, uint32_t headDim, uint32_t waveSize = 32,
             bool reverse = false);

/// The unfused attention pieces, host pointers, synchronous (upload, one launch sequence, download); float32.
/// attentionScores: Q, K (B,S,H,D) -> scores (B,H,S,S) = scale Q K^T (shaders/attention-scores.glsl:33-65);
/// scale 0 means 1/sqrt(headDim).
void attentionScores(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* Q, const float* K,
                     float* scores, uint32_t batchSize, uint32_t seqLen, uint32_t numHeads, uint32_t headDim,
                     float scale = 0.0f);
/// Softmax over the last axis of (rows, features) (shaders/activation-softmax.glsl:34-84).
void softmax(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* input, float* output,
             size_t rows, uint32_t features);
/// weights (B,H,S,S) . V (B,S,H,D) -> (B,S,H,D); causal sums over k <= q only
/// (shaders/attention-output.glsl:28-70, attention-output-gpt.glsl:29-72).
void attentionOutput(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* weights, const float* V,
                     float* output, uint32_t batchSize, uint32_t seqLen, uint32_t numHeads, uint32_t headDim,
                     bool causal = false);
/// Backward of softmax(scale Q K^T) V: every tensor (B,H,S,D), attnWeights (B,H,S,S)
/// (shaders/attention-backward.glsl:73-195).
void attentionBackward(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* gradOutput,
                       const float* Q, const float* K, const float* V, const float* attnWeights, float* gradQ,
                       float* gradK, float* gradV, uint32_t batchSize, uint32_t numHeads, uint32_t seqLen,
                       uint32_t headDim, float scale = 0.0f);

}  // namespace ops
}  // namespace grilly

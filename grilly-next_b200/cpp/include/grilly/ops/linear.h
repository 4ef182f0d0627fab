#pragma once
// Linear projection output = x W^T + bias: the step before attention (Q/K/V projections, packed or separate) and
// after it (output projection).  Keeps the reference's call (cpp/include/grilly/ops/linear.h:31-56: LinearParams,
// host pointers in and out, synchronous); the extended form chooses the bf16 tensor-core kernel.
#include <cstdint>

#include "grilly/buffer_pool.h"
#include "grilly/command_batch.h"
#include "grilly/ops/attention.h"
#include "grilly/pipeline_cache.h"

namespace grilly {
namespace ops {

/// Push-constant block of fnn-linear.glsl, kept as the public parameter struct.
struct LinearParams {
    uint32_t batchSeq;
    uint32_t inputDim;
    uint32_t outputDim;
    uint32_t hasBias;
};

/// x (batchSeq, inputDim), weights (outputDim, inputDim), bias (outputDim) or nullptr, output (batchSeq, outputDim):
/// host float32, row-major.  Exact float32 arithmetic.
void linear(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* x, const float* weights,
            const float* bias, float* output, const LinearParams& p);

/// The same with a choice of arithmetic: Precision::BF16 rounds x and the weights to bf16 on the device and runs the
/// product on the tcgen05 tensor cores with float32 accumulation (inputDim must be a multiple of 8).
void linearEx(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* x, const float* weights,
              const float* bias, float* output, const LinearParams& p, Precision precision);

/// Fused QKV projection (shaders/fused-qkv-projection.glsl:40-74): wQKV is [W_q; W_k; W_v] of shape
/// (3 * numHeads * headDim, hiddenDim), bQKV the packed bias or nullptr; output (batchSeq, 3 * numHeads * headDim).
void fusedQKVProjection(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* x, const float* wQKV,
                        const float* bQKV, float* output, uint32_t batchSeq, uint32_t hiddenDim, uint32_t numHeads,
                        uint32_t headDim, Precision precision = Precision::FP32);

}  // namespace ops
}  // namespace grilly

#pragma once
// CPU reference of the fused MLA decompression + attention, the reference's
// experimental::fusedAttentionCPU (cpp/include/grilly/experimental/fused_attention.h:141-146,
// cpp/src/experimental/fused_attention.cpp:255-357).  It is a CPU function in the reference too (bound as
// grilly_core.fused_attention_cpu, no Device argument): a verification aid for the latent path, not a fallback
// of any GPU op.
#include <cstdint>

namespace grilly {
namespace experimental {

/// Q, output: (batch, heads, seqLen, headDim); latents: (cachedTokens * heads, latentDim); wUp: (latentDim,
/// 2 * headDim), decoding to [K | V]; mask: nullptr or additive (batch, seqLen, cachedTokens); scale 0 => 1/sqrt(D).
void fusedAttentionCPU(const float* Q, const float* latents, const float* wUp, const float* mask, float* output,
                       uint32_t batchSize, uint32_t seqLen, uint32_t cachedTokens, uint32_t numHeads,
                       uint32_t headDim, uint32_t latentDim, float scale = 0.0f);

}  // namespace experimental
}  // namespace grilly

// fusedAttentionCPU: decode the latents with W_up, then plain softmax attention, on the host.
#include <algorithm>
#include <cmath>
#include <vector>

#include "grilly/experimental/fused_attention.h"

namespace grilly {
namespace experimental {

void fusedAttentionCPU(const float* Q, const float* latents, const float* wUp, const float* mask, float* output,
                       uint32_t B, uint32_t S, uint32_t T, uint32_t H, uint32_t D, uint32_t L, float scale) {
    if (scale == 0.0f) scale = 1.0f / std::sqrt(float(D));
    const size_t rows = size_t(T) * H, wide = size_t(2) * D;
    // step 1: [K | V] rows = latents W_up
    std::vector<float> kv(rows * wide);
    for (size_t r = 0; r < rows; ++r)
        for (size_t j = 0; j < wide; ++j) {
            float sum = 0.0f;
            for (uint32_t l = 0; l < L; ++l) sum += latents[r * L + l] * wUp[size_t(l) * wide + j];
            kv[r * wide + j] = sum;
        }
    // step 2: per (batch, head, query): scores over the T cached tokens (K and V are shared by the batch)
    std::vector<float> scores(std::max<uint32_t>(T, 1));
    for (uint32_t b = 0; b < B; ++b)
        for (uint32_t h = 0; h < H; ++h)
            for (uint32_t q = 0; q < S; ++q) {
                const size_t qo = ((size_t(b) * H + h) * S + q) * D;
                float top = -1e30f;
                for (uint32_t t = 0; t < T; ++t) {
                    const float* kr = &kv[(size_t(t) * H + h) * wide];
                    float dot = 0.0f;
                    for (uint32_t d = 0; d < D; ++d) dot += Q[qo + d] * kr[d];
                    float s = dot * scale;
                    if (mask) s += mask[(size_t(b) * S + q) * T + t];
                    scores[t] = s;
                    top = std::max(top, s);
                }
                float total = 0.0f;
                for (uint32_t t = 0; t < T; ++t) { scores[t] = std::exp(scores[t] - top); total += scores[t]; }
                for (uint32_t t = 0; t < T; ++t) scores[t] /= total;
                float* o = output + qo;
                std::fill(o, o + D, 0.0f);
                for (uint32_t t = 0; t < T; ++t) {
                    const float* vr = &kv[(size_t(t) * H + h) * wide + D];
                    for (uint32_t d = 0; d < D; ++d) o[d] += scores[t] * vr[d];
                }
            }
}

}  // namespace experimental
}  // namespace grilly

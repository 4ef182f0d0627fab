// Standalone RoPE and attention-mask ops (element-wise, HBM-bound).  Replace shaders/rope.glsl
// and shaders/attention-mask.glsl; inside the attention kernels the same arithmetic is fused.
#include "common.cuh"

namespace grl {

// One thread per rotation pair of x (B,S,H,D): reads two values, writes two.
__global__ void rope_kernel(const float* __restrict__ x, float* __restrict__ y, size_t n_pairs, int S, int H,
                            int D, int mode, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            RopeFreq f) {
    const int half = D / 2;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n_pairs;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int j = (int)(idx % half);
        const size_t vec = idx / half;             // (b*S + s)*H + h
        const int s = (int)((vec / H) % S);
        float c, sn;
        if (cos_t) {  // rope.glsl:109-113
            c = cos_t[(size_t)s * half + j];
            sn = sin_t[(size_t)s * half + j];
        } else {
            rope_sincos(s, f.inv_freq[j], &c, &sn);
        }
        const int d0 = (mode == GRL_ROPE_INTERLEAVED) ? 2 * j : j;
        const int d1 = (mode == GRL_ROPE_INTERLEAVED) ? 2 * j + 1 : j + half;
        const float x0 = x[vec * D + d0], x1 = x[vec * D + d1];
        y[vec * D + d0] = x0 * c - x1 * sn;   // rope.glsl:76-125: x*cos + rotate_half(x)*sin
        y[vec * D + d1] = x1 * c + x0 * sn;
    }
}

__global__ void attention_mask_kernel(float* __restrict__ scores, const float* __restrict__ key_mask, size_t total,
                                      int H, int S, int causal, float mask_value) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int k = (int)(idx % S);
        const int q = (int)((idx / S) % S);
        if (causal) {
            if (k > q) scores[idx] = mask_value;           // attention-mask.glsl:42-46
        } else {
            const size_t b = idx / ((size_t)H * S * S);
            if (key_mask[b * S + k] < 0.5f) scores[idx] = mask_value;  // :47-54
        }
    }
}

}  // namespace grl

using namespace grl;

extern "C" {

int grl_rope(grl_device* dev, const float* x, float* y, int batch, int seq_len, int heads, int head_dim,
             float base, float scaling, int mode, const float* cos_table, const float* sin_table) {
    GRL_REQUIRE(dev && x && y, "NULL argument");
    GRL_REQUIRE(batch > 0 && seq_len > 0 && heads > 0, "bad shape");
    GRL_REQUIRE(head_dim > 0 && head_dim % 2 == 0 && head_dim <= 256, "head_dim must be even and <= 256");
    GRL_REQUIRE(mode == GRL_ROPE_INTERLEAVED || mode == GRL_ROPE_HALF, "unknown rope mode");
    GRL_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "cos and sin tables go together");
    DeviceGuard g(dev->ordinal);
    const size_t n_pairs = (size_t)batch * seq_len * heads * (head_dim / 2);
    int blocks = (int)((n_pairs + 255) / 256 < (size_t)dev->prop.multiProcessorCount * 32
                           ? (n_pairs + 255) / 256
                           : (size_t)dev->prop.multiProcessorCount * 32);
    rope_kernel<<<blocks, 256, 0, dev->stream>>>(x, y, n_pairs, seq_len, heads, head_dim, mode, cos_table,
                                                 sin_table, make_rope_freq(head_dim, base, scaling));
    GRL_LAUNCHED("rope_kernel");
    return GRL_OK;
}

int grl_attention_mask(grl_device* dev, float* scores, const float* key_mask, int batch, int heads,
                       int seq_len, int causal, float mask_value) {
    GRL_REQUIRE(dev && scores, "NULL argument");
    GRL_REQUIRE(batch > 0 && heads > 0 && seq_len > 0, "bad shape");
    GRL_REQUIRE(causal || key_mask, "a key mask is required when causal == 0");
    DeviceGuard g(dev->ordinal);
    const size_t total = (size_t)batch * heads * seq_len * seq_len;
    int blocks = (int)((total + 255) / 256 < (size_t)dev->prop.multiProcessorCount * 32
                           ? (total + 255) / 256
                           : (size_t)dev->prop.multiProcessorCount * 32);
    attention_mask_kernel<<<blocks, 256, 0, dev->stream>>>(scores, key_mask, total, heads, seq_len, causal,
                                                           mask_value);
    GRL_LAUNCHED("attention_mask_kernel");
    return GRL_OK;
}

}  // extern "C"

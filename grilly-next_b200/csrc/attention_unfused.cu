// The unfused attention pieces and the attention backward pass, for callers of the legacy three-step path.
//
// Replaces shaders/attention-scores.glsl (Q.K^T * scale into a (B,H,S,S) tensor), activation-softmax.glsl
// (three passes: row maximum, sum of exponentials, normalise), attention-output.glsl / attention-output-gpt.glsl
// (weights . V, the GPT form summing only over k <= q) and attention-backward.glsl (grad_V = A^T gO; grad_A = gO V^T;
// softmax backward; grad_Q, grad_K).  The fused kernels are the fast path; these exist so that code written against
// the separate shaders keeps working, and so that training code has a backward.  Every product is one strided,
// batched, shared-memory tiled float32 GEMM with the sum over the inner index in ascending order, as the
// shaders' loops run.
#include "common.cuh"

namespace grl {

struct GemmView {          // element (r, c) of batch (b, h) lives at base[b*sb + h*sh + r*sr + c*sc]
    const float* base;
    long long sb, sh, sr, sc;
};
struct GemmOut {
    float* base;
    long long sb, sh, sr, sc;
};

// C(m,n) = alpha * sum_k A(m,k) B(k,n), k ascending; causal_k != 0 limits the sum to k <= m (attention-output-gpt).
__global__ void __launch_bounds__(256) bgemm_kernel(GemmView A, GemmView B, GemmOut C, int M, int N, int K, int H,
                                                     float alpha, int causal_k) {
    __shared__ float As[16][17], Bs[16][17];
    const int lx = threadIdx.x & 15, ly = threadIdx.x >> 4;
    const int bh = blockIdx.z, b = bh / H, h = bh % H;
    const int m = blockIdx.y * 16 + ly, n = blockIdx.x * 16 + lx;
    const float* a = A.base + b * A.sb + h * A.sh;
    const float* bb = B.base + b * B.sb + h * B.sh;
    const int k_end = causal_k ? min(K, blockIdx.y * 16 + 16) : K;      // rows of this tile see k <= m only
    float acc = 0.f;
    for (int k0 = 0; k0 < k_end; k0 += 16) {
        As[ly][lx] = (m < M && k0 + lx < K) ? a[m * A.sr + (k0 + lx) * A.sc] : 0.f;
        Bs[ly][lx] = (n < N && k0 + ly < K) ? bb[(k0 + ly) * B.sr + n * B.sc] : 0.f;
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk)
            if (!causal_k || k0 + kk <= m) acc = fmaf(As[ly][kk], Bs[kk][lx], acc);
        __syncthreads();
    }
    if (m < M && n < N) C.base[b * C.sb + h * C.sh + m * C.sr + n * C.sc] = acc * alpha;
}

// Row-wise softmax of (rows, features): max from -1e10 as activation-softmax.glsl:34-84 starts it, exp(x - max) / sum.
__global__ void __launch_bounds__(256) softmax_rows_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                            size_t rows, int features) {
    __shared__ float red[8];
    const size_t row = blockIdx.x;
    if (row >= rows) return;
    const float* x = in + row * features;
    float* y = out + row * features;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float mx = -1e10f;
    for (int f = tid; f < features; f += 256) mx = fmaxf(mx, x[f]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float sum = 0.f;
    for (int f = tid; f < features; f += 256) sum += expf(x[f] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = 0.f;
    for (int w = 0; w < 8; ++w) sum += red[w];
    for (int f = tid; f < features; f += 256) y[f] = expf(x[f] - mx) / sum;
}

// grad_scores[i][j] = attn[i][j] * (grad_attn[i][j] - sum_k attn[i][k] grad_attn[i][k]), in place over grad_attn
// (attention-backward.glsl pass 2, the softmax backward; the scale goes into the two products that follow).
__global__ void __launch_bounds__(256) softmax_backward_rows_kernel(const float* __restrict__ attn, float* grad, size_t rows,
                                                                     int features) {
    __shared__ float red[8];
    const size_t row = blockIdx.x;
    if (row >= rows) return;
    const float* a = attn + row * features;
    float* g = grad + row * features;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float dot = 0.f;
    for (int f = tid; f < features; f += 256) dot = fmaf(a[f], g[f], dot);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) red[warp] = dot;
    __syncthreads();
    dot = 0.f;
    for (int w = 0; w < 8; ++w) dot += red[w];
    for (int f = tid; f < features; f += 256) g[f] = a[f] * (g[f] - dot);
}

static int launch_bgemm(grl_device* dev, GemmView A, GemmView B, GemmOut C, int M, int N, int K, int batch, int H,
                        float alpha, int causal_k) {
    dim3 grid((N + 15) / 16, (M + 15) / 16, batch * H);
    bgemm_kernel<<<grid, 256, 0, dev->stream>>>(A, B, C, M, N, K, H, alpha, causal_k);
    GRL_LAUNCHED("bgemm_kernel");
    return GRL_OK;
}

}  // namespace grl

using namespace grl;

extern "C" {

int grl_attention_scores(grl_device* dev, const float* q, const float* k, float* scores, int batch, int seq_len, int heads,
                         int head_dim, float scale) {
    GRL_REQUIRE(dev && q && k && scores, "NULL argument");
    GRL_REQUIRE(batch > 0 && seq_len > 0 && heads > 0 && head_dim > 0, "bad shape");
    DeviceGuard g(dev->ordinal);
    const long long S = seq_len, H = heads, D = head_dim;
    if (scale == 0.f) scale = 1.f / sqrtf((float)head_dim);
    // Q, K: (B,S,H,D); scores (B,H,S,S)
    GemmView A{q, S * H * D, D, H * D, 1}, B{k, S * H * D, D, 1, H * D};
    GemmOut C{scores, H * S * S, S * S, S, 1};
    return launch_bgemm(dev, A, B, C, seq_len, seq_len, head_dim, batch, heads, scale, 0);
}

int grl_softmax(grl_device* dev, const float* in, float* out, size_t rows, int features) {
    GRL_REQUIRE(dev && in && out, "NULL argument");
    GRL_REQUIRE(rows > 0 && features > 0, "bad shape");
    GRL_REQUIRE(rows <= 0x7fffffffull, "too many rows");
    DeviceGuard g(dev->ordinal);
    softmax_rows_kernel<<<(unsigned)rows, 256, 0, dev->stream>>>(in, out, rows, features);
    GRL_LAUNCHED("softmax_rows_kernel");
    return GRL_OK;
}

int grl_attention_output(grl_device* dev, const float* weights, const float* v, float* out, int batch, int seq_len,
                         int heads, int head_dim, int causal) {
    GRL_REQUIRE(dev && weights && v && out, "NULL argument");
    GRL_REQUIRE(batch > 0 && seq_len > 0 && heads > 0 && head_dim > 0, "bad shape");
    DeviceGuard g(dev->ordinal);
    const long long S = seq_len, H = heads, D = head_dim;
    // weights (B,H,S,S); V, out (B,S,H,D)
    GemmView A{weights, H * S * S, S * S, S, 1}, B{v, S * H * D, D, H * D, 1};
    GemmOut C{out, S * H * D, D, H * D, 1};
    return launch_bgemm(dev, A, B, C, seq_len, head_dim, seq_len, batch, heads, 1.f, causal ? 1 : 0);
}

int grl_attention_backward(grl_device* dev, const float* grad_out, const float* q, const float* k, const float* v,
                           const float* attn, float* grad_q, float* grad_k, float* grad_v, float* scratch, int batch,
                           int heads, int seq_len, int head_dim, float scale) {
    GRL_REQUIRE(dev && grad_out && q && k && v && attn && grad_q && grad_k && grad_v && scratch, "NULL argument");
    GRL_REQUIRE(batch > 0 && seq_len > 0 && heads > 0 && head_dim > 0, "bad shape");
    DeviceGuard g(dev->ordinal);
    const long long S = seq_len, H = heads, D = head_dim;
    if (scale == 0.f) scale = 1.f / sqrtf((float)head_dim);
    // all of Q, K, V, grad_out and the three gradients: (B,H,S,D); attn, scratch: (B,H,S,S)
    const long long qb = H * S * D, qh = S * D, ab = H * S * S, ah = S * S;
    // pass 0: grad_V[j][d] = sum_i attn[i][j] grad_out[i][d]
    int rc = launch_bgemm(dev, GemmView{attn, ab, ah, 1, S}, GemmView{grad_out, qb, qh, D, 1}, GemmOut{grad_v, qb, qh, D, 1},
                          seq_len, head_dim, seq_len, batch, heads, 1.f, 0);
    // pass 1: grad_attn[i][j] = sum_d grad_out[i][d] V[j][d]  -> scratch
    if (!rc) rc = launch_bgemm(dev, GemmView{grad_out, qb, qh, D, 1}, GemmView{v, qb, qh, 1, D}, GemmOut{scratch, ab, ah, S, 1},
                               seq_len, seq_len, head_dim, batch, heads, 1.f, 0);
    if (rc) return rc;
    // softmax backward, row by row, in place over scratch
    const size_t rows = (size_t)batch * heads * seq_len;
    GRL_REQUIRE(rows <= 0x7fffffffull, "too many rows");
    softmax_backward_rows_kernel<<<(unsigned)rows, 256, 0, dev->stream>>>(attn, scratch, rows, seq_len);
    GRL_LAUNCHED("softmax_backward_rows_kernel");
    // pass 2: grad_Q[i][d] = scale * sum_j gS[i][j] K[j][d];  grad_K[j][d] = scale * sum_i gS[i][j] Q[i][d]
    rc = launch_bgemm(dev, GemmView{scratch, ab, ah, S, 1}, GemmView{k, qb, qh, D, 1}, GemmOut{grad_q, qb, qh, D, 1}, seq_len,
                      head_dim, seq_len, batch, heads, scale, 0);
    if (!rc) rc = launch_bgemm(dev, GemmView{scratch, ab, ah, 1, S}, GemmView{q, qb, qh, D, 1}, GemmOut{grad_k, qb, qh, D, 1},
                               seq_len, head_dim, seq_len, batch, heads, scale, 0);
    return rc;
}

}  // extern "C"

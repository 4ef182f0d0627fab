// fp32 SIMT flash-attention forward (exact path, max-abs <= 1e-4 against the fp32 oracle).
//
// Replaces the three-pass dispatch of ops::flashAttention2 (cpp/src/ops/attention.cpp:112-152)
// and the per-(q,k)-thread shaders flash-attention2.glsl / flash-attention2-rope.glsl with ONE
// launch: a CTA owns 64 query rows of one (batch, head), streams 64-key K/V tiles through
// shared memory, keeps running max / sum / accumulator in registers (online softmax) and
// writes O once.  Covers every mask convention of the reference, causal and ragged lengths
// as predicates (no S x S tensor), both RoPE pairings applied while the Q/K tiles are loaded.
#include "common.cuh"

namespace grl {

constexpr int FM = 64;   // query rows per CTA
constexpr int FN = 64;   // keys per tile
constexpr float kExcluded = -1e30f;

struct FlashF32Args {
    const void* q;
    const void* k;
    const void* v;
    void* o;
    int B, H, S, D;
    float scale;
    int causal;
    const int32_t* seq_lens;
    const float* mask;
    int mask_kind;
    int rope_mode;
    const float2* rope;  // (S, D/2) cos/sin or NULL
};

template <typename TIn, int D>
__device__ __forceinline__ void load_tile(float* dst /*[64][D+4]*/, const TIn* src, int row0, int n_valid_rows,
                                          int rope_mode, const float2* rope, int tid) {
    constexpr int LD = D + 4;
    if (rope_mode == GRL_ROPE_NONE) {
        for (int idx = tid; idx < 64 * D; idx += 256) {
            int r = idx / D, d = idx % D;
            float x = 0.f;
            if (r < n_valid_rows) x = load_as_float<TIn>(src + (size_t)(row0 + r) * D + d);
            dst[r * LD + d] = x;
        }
    } else {
        constexpr int HALF = D / 2;
        for (int idx = tid; idx < 64 * HALF; idx += 256) {
            int r = idx / HALF, i = idx % HALF;
            int d0 = (rope_mode == GRL_ROPE_INTERLEAVED) ? 2 * i : i;
            int d1 = (rope_mode == GRL_ROPE_INTERLEAVED) ? 2 * i + 1 : i + HALF;
            float y0 = 0.f, y1 = 0.f;
            if (r < n_valid_rows) {
                const TIn* p = src + (size_t)(row0 + r) * D;
                float x0 = load_as_float<TIn>(p + d0), x1 = load_as_float<TIn>(p + d1);
                float2 cs = rope[(size_t)(row0 + r) * HALF + i];
                y0 = x0 * cs.x - x1 * cs.y;
                y1 = x0 * cs.y + x1 * cs.x;
            }
            dst[r * LD + d0] = y0;
            dst[r * LD + d1] = y1;
        }
    }
}

template <typename TIn, typename TOut, int D>
__global__ void __launch_bounds__(256) flash_fwd_f32_kernel(FlashF32Args a) {
    constexpr int LD = D + 4;
    constexpr int DPT = D / 16;  // output columns per thread
    extern __shared__ __align__(16) float smem[];
    float* Qs = smem;
    float* Ks = Qs + FM * LD;
    float* Vs = Ks + FN * LD;
    float* Ps = Vs + FN * LD;  // [64][FN+4]
    constexpr int LP = FN + 4;

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int n_qt = gridDim.x;
    const int qt = a.causal ? (n_qt - 1 - blockIdx.x) : blockIdx.x;  // heavy tiles first
    const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int S = a.S;
    const int q0 = qt * FM;
    const int len = a.seq_lens ? min(a.seq_lens[b], S) : S;
    const size_t base = (size_t)bh * S * D;
    TOut* O = reinterpret_cast<TOut*>(a.o) + base;

    if (q0 >= len) {  // padded query rows are defined as zero
        for (int idx = tid; idx < FM * D; idx += 256) {
            int r = idx / D;
            if (q0 + r < S) store_from_float<TOut>(O + (size_t)(q0 + r) * D + idx % D, 0.f);
        }
        return;
    }
    const TIn* Q = reinterpret_cast<const TIn*>(a.q) + base;
    const TIn* K = reinterpret_cast<const TIn*>(a.k) + base;
    const TIn* V = reinterpret_cast<const TIn*>(a.v) + base;

    load_tile<TIn, D>(Qs, Q, q0, min(FM, S - q0), a.rope_mode, a.rope, tid);

    float m[4], l[4], acc[4][DPT];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        m[r] = kExcluded;
        l[r] = 0.f;
#pragma unroll
        for (int e = 0; e < DPT; ++e) acc[r][e] = 0.f;
    }

    int k_end = len;
    if (a.causal) k_end = min(k_end, q0 + FM);
    const int n_kt = (k_end + FN - 1) / FN;

    for (int kt = 0; kt < n_kt; ++kt) {
        const int k0 = kt * FN;
        __syncthreads();  // previous tile's Ks/Vs/Ps fully consumed
        load_tile<TIn, D>(Ks, K, k0, min(FN, S - k0), a.rope_mode, a.rope, tid);
        load_tile<TIn, D>(Vs, V, k0, min(FN, S - k0), GRL_ROPE_NONE, nullptr, tid);
        __syncthreads();

        float s[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[r][c] = 0.f;
#pragma unroll 4
        for (int d = 0; d < D; d += 4) {
            float4 qv[4], kv[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) qv[r] = *reinterpret_cast<const float4*>(&Qs[(ty * 4 + r) * LD + d]);
#pragma unroll
            for (int c = 0; c < 4; ++c) kv[c] = *reinterpret_cast<const float4*>(&Ks[(tx + 16 * c) * LD + d]);
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    s[r][c] = fmaf(qv[r].x, kv[c].x, s[r][c]);
                    s[r][c] = fmaf(qv[r].y, kv[c].y, s[r][c]);
                    s[r][c] = fmaf(qv[r].z, kv[c].z, s[r][c]);
                    s[r][c] = fmaf(qv[r].w, kv[c].w, s[r][c]);
                }
        }

#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int qi = q0 + ty * 4 + r;
            float mx = kExcluded;
            bool valid[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int kj = k0 + tx + 16 * c;
                bool ok = (kj < len) && (qi < S) && (!a.causal || kj <= qi);
                float sc = s[r][c] * a.scale;
                if (ok && a.mask_kind != GRL_MASK_NONE) {
                    float mv;
                    if (a.mask_kind == GRL_MASK_KEY) mv = a.mask[(size_t)b * S + kj];
                    else if (a.mask_kind == GRL_MASK_BSS) mv = a.mask[((size_t)b * S + qi) * S + kj];
                    else mv = a.mask[(((size_t)b * a.H + h) * S + qi) * S + kj];
                    if (!(mv > 0.f)) sc = -1e9f;  // replaced, not added (tests/test_attention.py:30)
                }
                valid[c] = ok;
                s[r][c] = sc;
                if (ok) mx = fmaxf(mx, sc);
            }
#pragma unroll
            for (int off = 1; off < 16; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float m_new = fmaxf(m[r], mx);
            float rs = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float p = valid[c] ? expf(s[r][c] - m_new) : 0.f;
                rs += p;
                Ps[(ty * 4 + r) * LP + tx + 16 * c] = p;
            }
#pragma unroll
            for (int off = 1; off < 16; off <<= 1) rs += __shfl_xor_sync(0xffffffffu, rs, off);
            const float corr = expf(m[r] - m_new);  // both finite (kExcluded is finite)
            l[r] = l[r] * corr + rs;
            m[r] = m_new;
#pragma unroll
            for (int e = 0; e < DPT; ++e) acc[r][e] *= corr;
        }
        __syncthreads();

#pragma unroll 4
        for (int kk = 0; kk < FN; ++kk) {
            float pv[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) pv[r] = Ps[(ty * 4 + r) * LP + kk];
#pragma unroll
            for (int e = 0; e < DPT; ++e) {
                // columns tx*4 + (e%4) + 64*(e/4) for D>=64; tx*DPT + e for D=32
                const int d = (DPT >= 4) ? (tx * 4 + (e & 3) + 64 * (e >> 2)) : (tx * DPT + e);
                const float vv = Vs[kk * LD + d];
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[r][e] = fmaf(pv[r], vv, acc[r][e]);
            }
        }
    }

#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int qi = q0 + ty * 4 + r;
        if (qi >= S) continue;
        const bool zero = (qi >= len) || !(l[r] > 0.f);
        const float inv = zero ? 0.f : 1.f / l[r];
#pragma unroll
        for (int e = 0; e < DPT; ++e) {
            const int d = (DPT >= 4) ? (tx * 4 + (e & 3) + 64 * (e >> 2)) : (tx * DPT + e);
            store_from_float<TOut>(O + (size_t)qi * D + d, acc[r][e] * inv);
        }
    }
}

template <typename TIn, typename TOut, int D>
static int launch_f32(grl_device* dev, const FlashF32Args& a) {
    constexpr size_t smem = sizeof(float) * (size_t)(3 * 64 * (D + 4) + 64 * (FN + 4));
    auto kern = flash_fwd_f32_kernel<TIn, TOut, D>;
    GRL_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((a.S + FM - 1) / FM, a.B * a.H);
    kern<<<grid, 256, smem, dev->stream>>>(a);
    GRL_LAUNCHED("flash_fwd_f32_kernel");
    return GRL_OK;
}

template <typename TIn, typename TOut>
static int dispatch_d(grl_device* dev, const FlashF32Args& a) {
    switch (a.D) {
        case 32: return launch_f32<TIn, TOut, 32>(dev, a);
        case 64: return launch_f32<TIn, TOut, 64>(dev, a);
        case 128: return launch_f32<TIn, TOut, 128>(dev, a);
        default:
            return set_error(GRL_ERR_UNSUPPORTED, "head_dim %d not supported (32, 64 or 128)", a.D);
    }
}

int flash_fwd_simt(grl_device* dev, const grl_flash_params* p, float scale, const float2* rope) {
    GRL_REQUIRE((int64_t)p->batch * p->heads <= 65535, "batch*heads above 65535 (grid y dimension of the fp32 kernel)");
    FlashF32Args a{p->q, p->k, p->v, p->o, p->batch, p->heads, p->seq_len, p->head_dim, scale,
                   p->causal, p->seq_lens, p->mask, p->mask ? p->mask_kind : GRL_MASK_NONE,
                   p->rope_mode, rope};
    if (p->in_dtype == GRL_F32 && p->out_dtype == GRL_F32) return dispatch_d<float, float>(dev, a);
    if (p->in_dtype == GRL_BF16 && p->out_dtype == GRL_F32) return dispatch_d<__nv_bfloat16, float>(dev, a);
    if (p->in_dtype == GRL_BF16 && p->out_dtype == GRL_BF16)
        return dispatch_d<__nv_bfloat16, __nv_bfloat16>(dev, a);
    if (p->in_dtype == GRL_F32 && p->out_dtype == GRL_BF16) return dispatch_d<float, __nv_bfloat16>(dev, a);
    return set_error(GRL_ERR_INVALID, "unknown dtype");
}

}  // namespace grl
